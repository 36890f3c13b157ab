"""Token embedding and output head."""
from __future__ import annotations

import torch

from .base import MATRIX, TABLE, DeferredNorm, ParamSpec, Part, StateRequest, register_part


class TokenEmbedding(Part):
    """``x[i] = scale * table[token_i] (+ position_table[pos_i])`` into the fp32 residual stream
    (src/model.rs:285-295; ``scale`` is 1 there)."""
    graph_safe = True
    family = "embedding"
    kind = "token_embedding"

    def __init__(self, vocab_size: int, width: int, scale: float = 1.0):
        self.vocab_size = int(vocab_size)
        self.width = int(width)
        self.scale = float(scale)
        self.table = None

    def param_specs(self):
        return {"table": ParamSpec((self.vocab_size, self.width), TABLE)}

    def state_request(self):
        """Fixed-size per-sequence storage of the embedding (``ctx.state`` while it runs)."""
        return None

    def forward(self, ctx, position) -> torch.Tensor:
        lay = ctx.layout
        x = torch.empty((lay.n_rows, self.width), device=self.table.device, dtype=torch.float32)
        ctx.ops.embed_pos(lay.tokens, lay.row_pos, self.table, position.table, x, self.scale)
        return x


@register_part("embedding", "hashed_pair_embedding")
class HashedPairEmbedding(TokenEmbedding):
    """``x[i] = scale * table[token_i] + pair_table[b_i]``: beside the token's row, a row of a second
    table chosen by a hash of the token and the one before it in its sequence,
    ``b_i = (token_(i-1) * mul_prev + token_i * mul_cur) mod buckets``; a sequence's first token
    takes the table's last row (row ``buckets``).

    The token before a step's first one belongs to the sequence's state: one number per slot in
    the sequence's state row (token ids are whole numbers below 2^24, exact in fp32), written by
    the same kernel once the sequence's first row of the step has read it."""
    kind = "hashed_pair_embedding"

    def __init__(self, vocab_size: int, width: int, buckets: int, mul_prev: int, mul_cur: int,
                 scale: float = 1.0):
        super().__init__(vocab_size, width, scale)
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        if self.buckets < 1:
            raise ValueError("a hashed pair embedding needs at least one bucket")
        if self.vocab_size >= 1 << 24:
            raise ValueError("token ids beyond 2^24 do not fit the state row")
        self.pair_table = None

    def param_specs(self):
        return {**super().param_specs(),
                "pair_table": ParamSpec((self.buckets + 1, self.width), TABLE)}

    def state_request(self):
        return StateRequest(1)

    def forward(self, ctx, position) -> torch.Tensor:
        if position.table is not None:
            raise ValueError("a hashed pair embedding does not add a position table")
        lay = ctx.layout
        x = torch.empty((lay.n_rows, self.width), device=self.table.device, dtype=torch.float32)
        ctx.ops.embed_hashed(lay, self.table, self.pair_table, ctx.state, x, self.scale,
                             self.mul_prev, self.mul_cur, self.buckets)
        return x


class LMHead(Part):
    """``logits = h @ W.T`` without bias, fp32 result; ``W`` is the token embedding table when
    tied (src/model.rs:317-325)."""
    graph_safe = True
    family = "head"
    kind = "lm_head"

    def __init__(self, vocab_size: int, width: int, tied: bool):
        self.vocab_size = int(vocab_size)
        self.width = int(width)
        self.tied = bool(tied)
        self.weight = None

    def param_specs(self):
        if self.tied:
            return {}
        return {"weight": ParamSpec((self.vocab_size, self.width), MATRIX)}

    def tie(self, table: torch.Tensor) -> None:
        self.weight = table

    def forward(self, ctx, h) -> torch.Tensor:
        """``h``: activation rows, or a :class:`DeferredNorm` of fp32 rows."""
        norm = None
        if isinstance(h, DeferredNorm):
            h, norm = h.x, h.args
        logits = torch.empty((h.shape[0], self.vocab_size), device=h.device, dtype=torch.float32)
        ctx.ops.linear(h, self.weight, None, logits, 0, None, norm)
        return logits
