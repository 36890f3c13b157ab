"""Two mixers side by side on the same input, their normed results averaged."""
from __future__ import annotations

import torch

from .base import VECTOR, Mixer, ParamSpec, PartSpec, StateRequest, build_part, register_part


@register_part("mixer", "normed_pair")
class NormedPair(Mixer):
    """``left`` and ``right`` (any two mixers, given as part descriptions) read the same rows;
    each result is RMS-normed over the width with a weight of its own (``left_norm``,
    ``right_norm``; a plain weight) and the pair's result is ``coef`` times their sum.

    Each branch writes into an fp32 buffer of its own; one row pass norms both, adds the
    average to the stream and, when the arrangement asks for it, hands out the normed rows of
    the stream's next reader.  Storage: the pair asks for what its branches ask for, the paged
    stores one after the other and the fixed-size state side by side in one row (the left
    branch's numbers first); each branch sees its own part.
    """
    can_overwrite = False
    takes_next_norm = True       # `forward(..., then=norm)` returns that norm's rows of the stream

    def __init__(self, width: int, eps: float, left: PartSpec, right: PartSpec, coef: float = 0.5):
        self.width, self.eps, self.coef = int(width), float(eps), float(coef)
        self.left = build_part("mixer", left)
        self.right = build_part("mixer", right)
        self.graph_safe = bool(self.left.graph_safe and self.right.graph_safe)
        self.left_norm = self.right_norm = None
        # paged stores: every branch's own first, then its further ones, in the order asked
        self._stores = []           # (branch index, is_main)
        for b, part in enumerate((self.left, self.right)):
            if part.cache_request() is not None:
                self._stores.append((b, True, part.cache_request()))
            for r in part.extra_cache_requests():
                self._stores.append((b, False, r))
        self._state = [(p.state_request().n_elements if p.state_request() is not None else 0)
                       for p in (self.left, self.right)]

    def children(self):
        return {"left": self.left, "right": self.right}

    def param_specs(self):
        return {"left_norm": ParamSpec((self.width,), VECTOR),
                "right_norm": ParamSpec((self.width,), VECTOR)}

    def cache_request(self):
        return self._stores[0][2] if self._stores else None

    def extra_cache_requests(self):
        return tuple(s[2] for s in self._stores[1:])

    def state_request(self):
        total = sum(self._state)
        return StateRequest(total) if total else None

    def _branch(self, ctx, b: int, part, h, like):
        """Run one branch on its part of the pair's storage; returns its fp32 result."""
        views = ((ctx.kv,) if self._stores else ()) + tuple(ctx.kv_extra)
        mine = [(v, main) for v, (bb, main, _) in zip(views, self._stores) if bb == b]
        kv, extra, state, writes = ctx.kv, ctx.kv_extra, ctx.state, ctx.writes_cache
        ctx.kv = next((v for v, main in mine if main), None)
        ctx.kv_extra = tuple(v for v, main in mine if not main)
        lo = sum(self._state[:b])
        ctx.state = state[:, lo:lo + self._state[b]] if self._state[b] else None
        try:
            if getattr(part, "can_overwrite", False):
                y = torch.empty_like(like)
                part.forward(ctx, h, y, accumulate=False)
            else:
                y = torch.zeros_like(like)
                part.forward(ctx, h, y)
        finally:
            ctx.kv, ctx.kv_extra, ctx.state, ctx.writes_cache = kv, extra, state, writes
        return y

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor, then=None):
        """``then``: the norm in front of the stream's next reader; its rows are returned."""
        a = self._branch(ctx, 0, self.left, h, residual)
        b = self._branch(ctx, 1, self.right, h, residual)
        nxt = None
        if then is not None:
            nxt = torch.empty(residual.shape, device=residual.device, dtype=ctx.rt.act_dtype)
        ctx.ops.rms_pair_add(a, self.left_norm, b, self.right_norm, self.eps, self.coef, residual,
                             then.weight if then is not None else None,
                             then.eps if then is not None else 0.0, nxt)
        return nxt
