"""Normalisation parts."""
from __future__ import annotations

import torch

from .base import VECTOR, DeferredNorm, Norm, ParamSpec, register_part


@register_part("norm", "layernorm")
class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * weight + bias`` per row with biased variance, statistics
    in fp32 (src/ops.rs:32-40).  Weight and bias are both required (src/engine.rs:141-152), unless
    ``bias=False``: a layer norm with a weight and no shift."""
    graph_safe = True

    def __init__(self, width: int, eps: float, bias: bool = True):
        self.width = int(width)
        self.eps = float(eps)
        self.has_bias = bool(bias)
        self.weight = None
        self.bias = None

    def param_specs(self):
        specs = {"weight": ParamSpec((self.width,), VECTOR)}
        if self.has_bias:
            specs["bias"] = ParamSpec((self.width,), VECTOR)
        return specs

    def add_into(self, ctx, y, residual, then: "LayerNorm | None" = None, rounded: bool = False):
        """``residual += norm(y)`` for a sublayer's fp32 result ``y`` in one pass over the rows,
        which can also hand out ``then(residual)`` (the norm in front of the next sublayer) and,
        with ``rounded``, the stream's rows in the activation type; the interface of
        :meth:`RMSNorm.add_into`.  Only for norms without a shift."""
        if self.has_bias or (then is not None and getattr(then, "has_bias", True)):
            raise ValueError("add_into: only layer norms without a shift are added in one pass")
        act = ctx.rt.act_dtype
        nxt = torch.empty(residual.shape, device=y.device, dtype=act) if then is not None else None
        cast = torch.empty(residual.shape, device=y.device, dtype=act) if rounded else None
        ctx.ops.ln_add(y, self.weight, self.eps, residual,
                       then.weight if then is not None else None,
                       then.eps if then is not None else 0.0, nxt, cast)
        return nxt, cast

    def defer(self, ctx, x):
        return DeferredNorm(ctx, self, x, (self.weight, self.bias, self.eps, ctx.rt.act_dtype))

    def forward(self, ctx, x, rows=None, n_rows=None):
        n = x.shape[0] if rows is None else (rows.numel() if n_rows is None else n_rows)
        out = torch.empty((n, self.width), device=x.device, dtype=ctx.rt.act_dtype)
        ctx.ops.layernorm(x, self.weight, self.bias, self.eps, out, rows)
        return out


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """``x / sqrt(mean(x^2) + eps) * weight`` per row, statistics and scaling in fp32 (``eps``
    inside the root).  No kernel folds this norm into the product that follows, so it never
    defers: one launch gives the rows to every reader."""
    graph_safe = True

    def __init__(self, width: int, eps: float, gain: float = 1.0):
        """``gain``: a constant that multiplies the result (a model that scales its logits does
        so through its last norm); folded into the weight when it is bound."""
        self.width = int(width)
        self.eps = float(eps)
        self.gain = float(gain)
        self.weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.width,), VECTOR)}

    def bind(self, params, runtime) -> None:
        super().bind(params, runtime)
        if self.gain != 1.0 and self.weight is not None:
            self.weight = (self.weight * self.gain).contiguous()

    def forward(self, ctx, x, rows=None, n_rows=None):
        n = x.shape[0] if rows is None else (rows.numel() if n_rows is None else n_rows)
        out = torch.empty((n, self.width), device=x.device, dtype=ctx.rt.act_dtype)
        ctx.ops.rmsnorm(x, self.weight, self.eps, out, rows)
        return out

    def add_into(self, ctx, y, residual, then: "RMSNorm | None" = None, rounded: bool = False):
        """``residual += norm(y)`` for a sublayer's fp32 result ``y``, in one pass over the rows
        that can also hand out what the next reader of the stream wants: with ``then`` the
        rows of ``then(residual)`` (the norm in front of the next sublayer), with ``rounded``
        the stream's rows in the activation type.  Returns ``(then's rows or None, rounded
        rows or None)``."""
        act = ctx.rt.act_dtype
        nxt = torch.empty(residual.shape, device=y.device, dtype=act) if then is not None else None
        cast = torch.empty(residual.shape, device=y.device, dtype=act) if rounded else None
        ctx.ops.rms_add(y, self.weight, self.eps, residual,
                        then.weight if then is not None else None,
                        then.eps if then is not None else 0.0, nxt, cast)
        return nxt, cast
