"""Linear attention with a fixed decay per head and a gated, normed output."""
from __future__ import annotations

import torch

from ..csrc.ops import ACT_NONE, ACT_SILU
from .base import VECTOR, Mixer, ParamSpec, StateRequest, register_part
from .linear import Linear


@register_part("mixer", "decayed_linear_attention")
class DecayedLinearAttention(Mixer):
    """``q, k = silu(Wq h), silu(Wk h)`` (``n_heads`` heads of ``head_dim``), ``v = silu(Wv h)``
    (heads of ``value_dim``).  Per head a state ``S`` (``head_dim x value_dim``, fp32, zero at a
    sequence's start):

        S_t = decay_h S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t        (no other scale)

    The heads' ``o`` side by side are RMS-normed together with the weight ``norm``, multiplied
    by ``sigmoid(Wg h)`` and mapped back by ``Wo``.

    How it runs: one product gives ``[q | k | v | g]`` in fp32; one kernel walks each sequence's
    tokens in order with the state in registers (silu applied as the rows are staged) and leaves
    the state in the sequence's state row; a row pass norms and gates.  Nothing grows with the
    sequence.
    """
    graph_safe = True
    can_overwrite = True

    def __init__(self, width: int, n_heads: int, head_dim: int, decay, eps: float,
                 value_dim: int | None = None):
        self.width, self.n_heads, self.head_dim = int(width), int(n_heads), int(head_dim)
        self.value_dim = int(value_dim) if value_dim else self.head_dim
        self.eps = float(eps)
        self.decay_host = torch.tensor([float(x) for x in decay], dtype=torch.float32)
        if self.decay_host.numel() != self.n_heads:
            raise ValueError(f"{self.n_heads} heads need {self.n_heads} decays, "
                             f"got {self.decay_host.numel()}")
        qk, vw = self.n_heads * self.head_dim, self.n_heads * self.value_dim
        self.col_q, self.col_k, self.col_v, self.col_g = 0, qk, 2 * qk, 2 * qk + vw
        self.v_width = vw
        self.proj = Linear(self.width, -(-(2 * qk + 2 * vw) // 8) * 8, bias=False)
        self.out = Linear(vw, self.width, bias=False)
        self.norm = self.decay = None

    def children(self):
        return {"proj": self.proj, "out": self.out}

    def param_specs(self):
        return {"norm": ParamSpec((self.v_width,), VECTOR)}

    def bind(self, params, runtime) -> None:
        super().bind(params, runtime)
        self.decay = self.decay_host.to(runtime.device)

    def state_request(self):
        return StateRequest(self.n_heads * self.head_dim * self.value_dim)

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True) -> None:
        lay, ops = ctx.layout, ctx.ops
        n, dev = lay.n_rows, h.device
        fused = self.proj(ctx, h, out_dtype=torch.float32)
        # the activation once per number, ahead of the recurrence: there every CTA of a head
        # stages the head's queries and keys, and would activate them again
        qkv = torch.empty((n, self.col_g), device=dev, dtype=torch.float32)
        ops.act_rows(fused, 0, ACT_SILU, None, qkv)
        o = torch.empty((n, self.v_width), device=dev, dtype=torch.float32)
        ops.linear_attention(qkv, self.col_q, self.col_k, self.col_v, ACT_NONE, self.decay,
                             ctx.state, lay, self.n_heads, self.head_dim, self.value_dim, o)
        y = torch.empty((n, self.v_width), device=dev, dtype=ctx.rt.act_dtype)
        ops.rmsnorm_gated(o, self.norm, fused, self.col_g, self.eps, y)
        if accumulate:
            self.out(ctx, y, residual=residual)
        else:
            self.out(ctx, y, out=residual)
