"""Grouped-query attention with rotated (and optionally normed) queries and keys, capped scores,
a mask by window or by block, a sink and a gate per head: each of them optional."""
from __future__ import annotations

import torch

from .base import VECTOR, KVRequest, Mixer, ParamSpec, register_part
from .linear import Linear
from .rotary import rotary_frequencies


@register_part("mixer", "masked_attention")
class MaskedAttention(Mixer):
    """``n_heads`` query heads over ``n_kv_heads`` key/value heads (query head ``h`` uses key head
    ``h // (n_heads / n_kv_heads)``), keys of ``head_dim`` numbers and values of ``value_dim``.

    One product gives ``[q | k | v | gate logits]`` in fp32 (no biases).  With ``qk_norm`` queries
    and keys get a per-head RMS norm (weights ``q_norm`` / ``k_norm`` of ``head_dim`` numbers,
    shared by the heads; ``eps`` inside the root), then, with ``rot_dims`` > 0, the first
    ``rot_dims`` numbers of every query and key head are turned by position, dimension ``i``
    paired with ``i + rot_dims / 2`` (``parts/rotary.py``); values get neither.

    A score is ``scale * q . k`` and, with ``softcap`` > 0, then ``softcap * tanh(score /
    softcap)``.  What position ``i`` sees among ``j <= i``:

    * ``window`` > 0: ``i - j < window``, and besides those every ``j < keep_first`` (the
      sequence's first tokens stay visible at their true positions);
    * ``chunk`` > 0: only ``j`` with ``floor(j / chunk) == floor(i / chunk)``, blocks counted from
      the sequence's position 0 whatever the step's cut;
    * neither: every ``j <= i``.

    With ``sink`` the softmax's denominator has one more term ``exp(sink_h)`` per head (no key, no
    value, neither scaled nor capped).  With ``gate`` head ``h``'s result is multiplied by
    ``sigmoid(Wg x)_h``, one logit per head from the mixer's own input.  ``Wo`` maps the
    concatenated heads back.

    Storage: keys and values of one size share a paged store of two planes, of different sizes
    they take two stores of one plane.  A store with a window gives back the pages that no later
    token sees, except those of the kept first tokens; a block mask never looks further back than
    ``chunk`` tokens, so its pages are given back like a window's.
    """
    graph_safe = True
    can_overwrite = True

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                 value_dim: int | None = None, eps: float = 1e-6, qk_norm: bool = False,
                 softcap: float = 0.0, window: int = 0, keep_first: int = 0, chunk: int = 0,
                 sink: bool = False, gate: bool = False, rot_dims: int = 0,
                 rot_base: float = 10000.0):
        self.width, self.n_heads, self.n_kv_heads = int(width), int(n_heads), int(n_kv_heads)
        self.head_dim = int(head_dim)
        self.value_dim = int(value_dim) if value_dim else self.head_dim
        self.one_store = self.value_dim == self.head_dim
        self.scale, self.eps, self.softcap = float(scale), float(eps), float(softcap or 0.0)
        self.window, self.keep_first, self.chunk = int(window), int(keep_first), int(chunk)
        if self.n_heads % self.n_kv_heads:
            raise ValueError("n_heads must be divisible by n_kv_heads")
        if self.window > 0 and self.chunk > 0:
            raise ValueError("a mask is a window or a block, not both")
        if self.window <= 0:
            self.keep_first = 0             # without a window every first token is seen anyway
        self.has_norm, self.has_sink, self.has_gate = bool(qk_norm), bool(sink), bool(gate)
        self.rot_dims = int(rot_dims)
        if self.rot_dims > self.head_dim:
            raise ValueError("more rotated dimensions than the head has")
        self.rot_freq_host = None if not self.rot_dims else \
            rotary_frequencies(self.rot_dims, rot_base, None)[0]
        self.rot_freq = None
        self.q_width = self.n_heads * self.head_dim
        self.k_width = self.n_kv_heads * self.head_dim
        self.v_width = self.n_kv_heads * self.value_dim
        self.col_k = self.q_width
        self.col_v = self.col_k + self.k_width
        self.col_gate = self.col_v + self.v_width
        outputs = self.col_gate + (self.n_heads if self.has_gate else 0)
        # rows of zeros fill the fused projection up to a multiple of 8 outputs
        self.proj = Linear(self.width, -(-outputs // 8) * 8, bias=False)
        self.out = Linear(self.n_heads * self.value_dim, self.width, bias=False)
        self.q_norm = self.k_norm = self.sink = None

    def children(self):
        return {"proj": self.proj, "out": self.out}

    def param_specs(self):
        specs = {}
        if self.has_norm:
            specs["q_norm"] = ParamSpec((self.head_dim,), VECTOR)
            specs["k_norm"] = ParamSpec((self.head_dim,), VECTOR)
        if self.has_sink:
            specs["sink"] = ParamSpec((self.n_heads,), VECTOR)
        return specs

    def bind(self, params, runtime) -> None:
        super().bind(params, runtime)
        if self.rot_freq_host is not None:
            self.rot_freq = self.rot_freq_host.to(runtime.device)

    def _look_back(self) -> int:
        return self.window if self.window > 0 else self.chunk

    def cache_request(self):
        return KVRequest(self.n_kv_heads, self.head_dim, self._look_back(),
                         planes=2 if self.one_store else 1, keep_first=self.keep_first)

    def extra_cache_requests(self):
        if self.one_store:
            return ()
        return (KVRequest(self.n_kv_heads, self.value_dim, self._look_back(), planes=1,
                          keep_first=self.keep_first),)

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True) -> None:
        lay, ops = ctx.layout, ctx.ops
        n, dev, act = lay.n_rows, h.device, ctx.rt.act_dtype
        keys = ctx.kv
        values = keys if self.one_store else ctx.kv_extra[0]
        fused = self.proj(ctx, h, out_dtype=torch.float32)
        q = torch.empty((n, self.q_width), device=dev, dtype=act)
        ops.qkv_norm_rope_append(fused, 0, self.col_k, self.col_v, self.q_norm, self.k_norm,
                                 self.eps, self.rot_freq, self.rot_dims, 1.0, lay, keys, values,
                                 self.n_heads, self.value_dim, q, ctx.writes_cache)
        attn = torch.empty((n, self.n_heads * self.value_dim), device=dev, dtype=act)
        ops.attention_masked(q, lay, keys, values, self.n_heads, self.sink, attn, self.scale,
                             self.softcap, self.window, self.keep_first, self.chunk,
                             fused if self.has_gate else None, self.col_gate)
        if accumulate:
            self.out(ctx, attn, residual=residual)
        else:
            self.out(ctx, attn, out=residual)
