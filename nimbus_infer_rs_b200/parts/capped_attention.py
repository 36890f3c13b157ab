"""Grouped-query attention with a short convolution on its projections, capped scores and a sink."""
from __future__ import annotations

import torch

from .base import VECTOR, KVRequest, Mixer, ParamSpec, StateRequest, register_part
from .linear import Linear
from .rotary import rotary_frequencies_by_wavelength


@register_part("mixer", "capped_attention")
class CappedAttention(Mixer):
    """``n_heads`` query heads over ``n_kv_heads`` key/value heads (query head ``h`` uses key head
    ``h // (n_heads / n_kv_heads)``), keys of ``head_dim`` numbers and values of ``value_dim``.

    ``q, k, v = Wq h, Wk h, Wv h`` (one fused product, fp32 result, no biases).  With ``conv`` =
    taps > 0 every channel of the three then passes a short causal convolution over time
    (weights ``[channels, taps]``, the last column on the current token, zeros before the
    sequence's start; no bias).  With ``rot_dims`` > 0 the first ``rot_dims`` numbers of every
    query and key head are turned by position, neighbouring numbers paired (``parts/rotary.py``).
    A score is ``scale * q . k`` and, with ``softcap`` > 0, then ``softcap * tanh(score /
    softcap)``; every earlier token and the token itself are seen; with ``sink`` the softmax's
    denominator has one more term ``exp(sink_h)`` per head, without key or value.

    Storage: keys and values of one size share a paged store of two planes (the layout of
    ``causal_attention``, whose decode and tensor-core prompt kernels then run, with cap and
    sink); of different sizes they take two stores of one plane.  In the sequence's state row, the last ``taps - 1`` projected rows (what the convolution of the next
    tokens reads of the past).
    """
    graph_safe = True
    can_overwrite = True

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                 value_dim: int | None = None, conv: int = 0, softcap: float = 0.0,
                 sink: bool = True, rot_dims: int = 0, rot_base: float = 10000.0,
                 rot_scaling: dict | None = None):
        self.width, self.n_heads, self.n_kv_heads = int(width), int(n_heads), int(n_kv_heads)
        self.head_dim = int(head_dim)
        self.value_dim = int(value_dim) if value_dim else self.head_dim
        self.one_store = self.value_dim == self.head_dim
        self.scale, self.softcap = float(scale), float(softcap or 0.0)
        self.taps = int(conv or 0)
        if self.n_heads % self.n_kv_heads:
            raise ValueError("n_heads must be divisible by n_kv_heads")
        self.has_sink = bool(sink)
        self.rot_dims = int(rot_dims)
        if self.rot_dims > self.head_dim:
            raise ValueError("more rotated dimensions than the head has")
        self.rot_freq_host = None if not self.rot_dims else \
            rotary_frequencies_by_wavelength(self.rot_dims, rot_base, rot_scaling)
        self.rot_freq = None
        self.q_width = self.n_heads * self.head_dim
        self.k_width = self.n_kv_heads * self.head_dim
        self.v_width = self.n_kv_heads * self.value_dim
        self.channels = self.q_width + self.k_width + self.v_width
        # rows of zeros fill the fused projection up to a multiple of 8 outputs
        self.proj = Linear(self.width, -(-self.channels // 8) * 8, bias=False)
        self.out = Linear(self.n_heads * self.value_dim, self.width, bias=False)
        self.conv = self.sink = None

    def children(self):
        return {"proj": self.proj, "out": self.out}

    def param_specs(self):
        specs = {}
        if self.taps > 0:
            specs["conv"] = ParamSpec((self.channels, self.taps), VECTOR)
        if self.has_sink:
            specs["sink"] = ParamSpec((self.n_heads,), VECTOR)
        return specs

    def bind(self, params, runtime) -> None:
        super().bind(params, runtime)
        if self.rot_freq_host is not None:
            self.rot_freq = self.rot_freq_host.to(runtime.device)

    def cache_request(self):
        return KVRequest(self.n_kv_heads, self.head_dim, 0, planes=2 if self.one_store else 1)

    def extra_cache_requests(self):
        return () if self.one_store else (KVRequest(self.n_kv_heads, self.value_dim, 0, planes=1),)

    def state_request(self):
        return StateRequest(max(self.taps - 1, 0) * self.channels)

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True) -> None:
        lay, ops = ctx.layout, ctx.ops
        n, dev, act = lay.n_rows, h.device, ctx.rt.act_dtype
        keys = ctx.kv
        values = keys if self.one_store else ctx.kv_extra[0]
        fused = self.proj(ctx, h, out_dtype=torch.float32)
        q = torch.empty((n, self.q_width), device=dev, dtype=act)
        ops.conv_rope_append(fused, 0, self.conv if self.taps > 0 else None, self.taps, ctx.state,
                             self.rot_freq, self.rot_dims, lay, keys, values, self.n_heads,
                             self.value_dim, q)
        attn = torch.empty((n, self.n_heads * self.value_dim), device=dev, dtype=act)
        ops.attention_capped(q, lay, keys, values, self.n_heads, self.sink, attn, self.scale,
                             self.softcap)
        if accumulate:
            self.out(ctx, attn, residual=residual)
        else:
            self.out(ctx, attn, out=residual)
