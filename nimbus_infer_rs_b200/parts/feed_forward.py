"""Per-token feed-forward parts."""
from __future__ import annotations

import torch

from ..csrc.ops import ACTIVATIONS, GLU_ACTIVATIONS, PARAM_ACTIVATIONS, ROW_ACTIVATIONS
from .base import VECTOR, FeedForward, ParamSpec, register_part
from .linear import Linear


@register_part("ffn", "dense_mlp")
class DenseMLP(FeedForward):
    """``residual += act(h @ Wfc + bfc) @ Wproj + bproj`` (src/model.rs:462-473,485-487).
    ``activation`` is ``gelu_tanh`` (src/ops.rs:21-24), ``gelu_erf`` or ``none``; ``hidden`` is
    a plain number, not derived from the width (src/config.rs:13).

    ``xielu`` is an activation with two learned numbers ``p, q`` (the parameter ``act``):
    ``z > 0: softplus(p) z^2 + z/2``; ``z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2``.
    The product kernels' epilogues carry no learned numbers, so the first product hands out
    fp32 rows and a pass of its own applies the activation to them."""
    graph_safe = True
    accepts_deferred_norm = True
    can_overwrite = True

    def __init__(self, width: int, hidden: int, activation: str, bias: bool = True):
        if activation not in ACTIVATIONS and activation not in ROW_ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r} "
                             f"(have {sorted({**ACTIVATIONS, **ROW_ACTIVATIONS})})")
        self.width, self.hidden = int(width), int(hidden)
        self.activation = activation
        self.learned = activation not in ACTIVATIONS
        self.act_code = ROW_ACTIVATIONS[activation] if self.learned else ACTIVATIONS[activation]
        self.fc = Linear(self.width, self.hidden, bias)
        self.proj = Linear(self.hidden, self.width, bias)
        self.act = None

    def children(self):
        return {"fc": self.fc, "proj": self.proj}

    def param_specs(self):
        return {"act": ParamSpec((2,), VECTOR)} if self.learned else {}

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True) -> None:
        if self.learned:
            z = self.fc(ctx, h, out_dtype=torch.float32)
            mid = torch.empty(z.shape, device=z.device, dtype=ctx.rt.act_dtype)
            ctx.ops.act_rows(z, 0, self.act_code, self.act, mid)
        else:
            mid = self.fc(ctx, h, act=self.act_code)
        if accumulate:
            self.proj(ctx, mid, residual=residual)
        else:
            self.proj(ctx, mid, out=residual)


@register_part("ffn", "gated_mlp")
class GatedMLP(FeedForward):
    """``residual += Wdown (act(Wgate h) * (Wup h))`` without biases; ``activation`` is ``relu``,
    ``silu``, ``gelu_tanh``, ``gelu_erf``, ``relu2`` or ``none``; or ``swish_clamp`` with its bound
    ``limit`` = L: ``g = min(Wgate h, L)``, ``u = clamp(Wup h, -L, L)``, and ``Wdown (g sigmoid(1.702
    g) (u + 1))``.

    One product gives ``[Wgate h | Wup h]`` side by side in fp32; a row pass applies the
    activation to the first half, multiplies by the second (both unrounded) and hands the
    product to ``Wdown`` in the activation type.

    ``extra_outputs`` > 0: that many more rows of weights ride on the first product for another
    reader of the same rows (a router beside a shared expert); their fp32 results are left in
    ``ctx.shared_projection`` as ``(rows, first column)``."""
    graph_safe = True
    can_overwrite = True

    def __init__(self, width: int, hidden: int, activation: str, limit: float | None = None,
                 extra_outputs: int = 0):
        if activation not in GLU_ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r} (have {sorted(GLU_ACTIVATIONS)})")
        if (limit is not None) != (activation in PARAM_ACTIVATIONS):
            raise ValueError(f"activation {activation!r} and limit={limit!r} do not go together")
        self.width, self.hidden = int(width), int(hidden)
        self.activation = activation
        self.act_param = float(limit) if limit is not None else 0.0
        self.act_code = GLU_ACTIVATIONS[activation]
        # the two halves start on multiples of 8 columns (fp32 rows on 32-byte boundaries)
        self.half = -(-self.hidden // 8) * 8
        self.extra_outputs = int(extra_outputs)
        self.fc = Linear(self.width, 2 * self.half + -(-self.extra_outputs // 8) * 8, bias=False)
        self.proj = Linear(self.hidden, self.width, bias=False)

    def children(self):
        return {"fc": self.fc, "proj": self.proj}

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True) -> None:
        both = self.fc(ctx, h, out_dtype=torch.float32)
        if self.extra_outputs:
            ctx.shared_projection = (both, 2 * self.half)
        mid = torch.empty((both.shape[0], self.hidden), device=both.device, dtype=ctx.rt.act_dtype)
        ctx.ops.glu_rows(both, 0, self.half, self.act_code, mid, self.act_param)
        if accumulate:
            self.proj(ctx, mid, residual=residual)
        else:
            self.proj(ctx, mid, out=residual)
