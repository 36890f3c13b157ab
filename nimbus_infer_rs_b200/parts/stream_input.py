"""Parts that act on the residual stream between layers."""
from __future__ import annotations

import torch

from .base import Part, register_part
from .linear import Linear


class StreamInput(Part):
    """Family ``stream``: ``forward(ctx, x, x0) -> x'`` runs right before a schedule entry and
    returns the stream that the entry's layer reads (``x0``: the embedding's output, kept
    unchanged through the step)."""
    family = "stream"


@register_part("stream", "embedding_remix")
class EmbeddingRemix(StreamInput):
    """``x <- W [x ; x0]``: the stream and the embedding's output side by side (``x`` first)
    through one matrix ``[width, 2 width]``, without bias.  The result is the new fp32 stream.

    The two rows are written side by side in the activation type (``x0``'s half once a step:
    it does not change) and one product maps them back."""
    graph_safe = True

    def __init__(self, width: int):
        self.width = int(width)
        self.proj = Linear(2 * self.width, self.width, bias=False)

    def children(self):
        return {"proj": self.proj}

    def forward(self, ctx, x: torch.Tensor, x0: torch.Tensor) -> torch.Tensor:
        pair = ctx.scratch.get(("embedding_remix", id(self)))
        if pair is None:
            pair = torch.empty((x.shape[0], 2 * self.width), device=x.device, dtype=ctx.rt.act_dtype)
            ctx.ops.cast_cols(x0, pair, self.width)
            ctx.scratch[("embedding_remix", id(self))] = pair
        ctx.ops.cast_cols(x, pair, 0)
        return self.proj(ctx, pair, out_dtype=torch.float32)
