"""A selective state-space mixer: a short convolution, then a scan whose decay and input follow
the token."""
from __future__ import annotations

import torch

from ..csrc.ops import ACT_SILU
from .base import VECTOR, Mixer, ParamSpec, StateRequest, register_part
from .linear import Linear


@register_part("mixer", "selective_scan")
class SelectiveScan(Mixer):
    """``[x | z] = W_in h`` (``inner`` channels each).  ``x`` passes a short causal convolution per
    channel (``conv`` ``[inner, taps]`` with bias ``conv_bias``, the last column on the current
    token, zeros before the sequence's start) and silu.  ``[dt | B | C] = W_x x`` (``dt_rank``,
    ``n_state``, ``n_state`` numbers); ``dt = softplus(W_dt dt + dt_bias)`` per channel; ``A =
    -exp(A_log)`` (``[inner, n_state]``).  Per channel ``c`` and state ``n``:

        S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n,     y_c = sum_n S[c, n] C_n + D_c x_c

    then ``y * silu(z)`` and ``W_o``.  The step sizes, decays, the state and its update are fp32.

    Storage, in the sequence's state row: the last ``taps - 1`` inputs of the convolution, then
    the state ``[inner, n_state]``.  Nothing grows with the sequence.
    """
    graph_safe = True
    can_overwrite = True

    def __init__(self, width: int, inner: int, n_state: int, dt_rank: int, conv: int = 0):
        self.width, self.inner = int(width), int(inner)
        self.n_state, self.dt_rank, self.taps = int(n_state), int(dt_rank), int(conv or 0)
        self.in_proj = Linear(self.width, 2 * self.inner, bias=False)
        self.low_width = self.dt_rank + 2 * self.n_state
        # rows of zeros fill the product up to a multiple of 8 outputs
        self.x_proj = Linear(self.inner, -(-self.low_width // 8) * 8, bias=False)
        self.dt_proj = Linear(self.dt_rank, self.inner, bias=False)
        self.out = Linear(self.inner, self.width, bias=False)
        self.conv = self.conv_bias = self.dt_bias = self.a_log = self.d_skip = None
        self.conv_floats = max(self.taps - 1, 0) * self.inner

    def children(self):
        return {"in_proj": self.in_proj, "x_proj": self.x_proj, "dt_proj": self.dt_proj,
                "out": self.out}

    def param_specs(self):
        specs = {"dt_bias": ParamSpec((self.inner,), VECTOR),
                 "a_log": ParamSpec((self.inner, self.n_state), VECTOR),
                 "d_skip": ParamSpec((self.inner,), VECTOR)}
        if self.taps > 0:
            specs["conv"] = ParamSpec((self.inner, self.taps), VECTOR)
            specs["conv_bias"] = ParamSpec((self.inner,), VECTOR, optional=True)
        return specs

    def state_request(self):
        return StateRequest(self.conv_floats + self.inner * self.n_state)

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True) -> None:
        lay, ops = ctx.layout, ctx.ops
        n, dev, act = lay.n_rows, h.device, ctx.rt.act_dtype
        xz = self.in_proj(ctx, h, out_dtype=torch.float32)
        x = torch.empty((n, self.inner), device=dev, dtype=torch.float32)
        x_act = x if act == torch.float32 else torch.empty((n, self.inner), device=dev, dtype=act)
        conv_state = ctx.state[:, :self.conv_floats] if self.conv_floats else None
        ops.conv_act(xz, 0, self.conv if self.taps > 0 else None,
                     self.conv_bias if self.taps > 0 else None, self.taps, ACT_SILU, conv_state,
                     lay, x, x_act)
        low = self.x_proj(ctx, x_act, out_dtype=torch.float32)
        dt_in = torch.empty((n, self.dt_rank), device=dev, dtype=act)
        ops.act_rows(low, 0, 0, None, dt_in)     # the step sizes' low-rank rows as an operand
        dt_lin = self.dt_proj(ctx, dt_in, out_dtype=torch.float32)
        y = torch.empty((n, self.inner), device=dev, dtype=act)
        ops.selective_scan(x, low, self.dt_rank, self.dt_rank + self.n_state, dt_lin, self.dt_bias,
                           self.a_log, self.d_skip, xz, self.inner, ctx.state[:, self.conv_floats:],
                           lay, self.n_state, y)
        if accumulate:
            self.out(ctx, y, residual=residual)
        else:
            self.out(ctx, y, out=residual)
