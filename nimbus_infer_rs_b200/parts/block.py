"""Arrangements of norms, mixer and feed-forward around the residual stream."""
from __future__ import annotations

import torch

from .base import Block, register_part


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    """``x += mixer(norm_mixer(x)); x += ffn(norm_ffn(x))`` (src/model.rs:297-300 with
    :345-357, :437-439, :448-460, :485-487).  ``x`` is the fp32 residual stream.  The
    feed-forward may be absent (then the layer is its first half).  A mixer that adds its result
    in a row pass of its own (``takes_next_norm``) is given the feed-forward's norm and hands
    back that norm's rows, computed in the same pass."""
    graph_safe = True

    def __init__(self):
        pass

    def forward(self, ctx, x, layer) -> None:
        mixer, ffn = layer.mixer, layer.ffn
        h = layer.norm_mixer.defer(ctx, x) if mixer.accepts_deferred_norm \
            else layer.norm_mixer.forward(ctx, x)
        if ffn is None:
            mixer.forward(ctx, h, x)
            return
        if getattr(mixer, "takes_next_norm", False) and hasattr(layer.norm_ffn, "add_into"):
            h = mixer.forward(ctx, h, x, then=layer.norm_ffn)
        else:
            mixer.forward(ctx, h, x)
            h = layer.norm_ffn.defer(ctx, x) if ffn.accepts_deferred_norm \
                else layer.norm_ffn.forward(ctx, x)
        ffn.forward(ctx, h, x)


@register_part("block", "parallel")
class ParallelBlock(Block):
    """``h = norm_mixer(x); x += mixer(h) + ffn(h)``: one norm, both sublayers read its output
    (the feed-forward may be absent).  Each sublayer adds into the fp32 stream; since neither
    reads the stream, the order of the two additions only changes the rounding."""
    graph_safe = True

    def __init__(self):
        pass

    def forward(self, ctx, x, layer) -> None:
        h = layer.norm_mixer.forward(ctx, x)
        layer.mixer.forward(ctx, h, x)
        if layer.ffn is not None:
            layer.ffn.forward(ctx, h, x)


@register_part("block", "sandwich")
class SandwichBlock(Block):
    """A norm before and after each sublayer: ``x += post_norm_mixer(mixer(norm_mixer(x)))``,
    then ``x += post_norm_ffn(ffn(norm_ffn(x)))`` (the feed-forward may be absent), then the
    layer's per-token input if it has one (``layer.side``), which reads the stream itself.

    A sublayer writes its result into an fp32 buffer of its own (a part that cannot overwrite
    gets zeros to add to); one pass over the rows norms that result, adds it to the stream and
    produces what the next reader wants: the next sublayer's normed rows, or the stream rounded
    to the activation type for the per-token input, or (``ctx.next_norm``) the normed rows the
    next layer's mixer reads, which that layer then finds in ``ctx.normed`` and does not compute
    again."""
    graph_safe = True
    takes_handed_norm = True

    def __init__(self):
        pass

    @staticmethod
    def _run(part, ctx, h, like):
        if getattr(part, "can_overwrite", False):
            y = torch.empty_like(like)
            part.forward(ctx, h, y, accumulate=False)
        else:
            y = torch.zeros_like(like)
            part.forward(ctx, h, y)
        return y

    def forward(self, ctx, x, layer) -> None:
        side = layer.side
        # the side input multiplies the stream by a matrix: in a 32-bit run the stream itself
        wants_rounded = side is not None and ctx.rt.act_dtype != torch.float32
        h, ctx.normed = ctx.normed, None
        if h is None:
            h = layer.norm_mixer.forward(ctx, x)
        y = self._run(layer.mixer, ctx, h, x)
        last = layer.post_norm_ffn if layer.ffn is not None else layer.post_norm_mixer
        # the next layer's first norm in the last pass: only if nothing changes the stream after
        # that pass, and the two norms are of one kind (one kernel norms both ways)
        then = ctx.next_norm if side is None and type(ctx.next_norm) is type(last) else None
        if layer.ffn is not None:
            h, _ = layer.post_norm_mixer.add_into(ctx, y, x, then=layer.norm_ffn)
            y = self._run(layer.ffn, ctx, h, x)
        ctx.normed, xr = last.add_into(ctx, y, x, then=then, rounded=wants_rounded)
        if side is not None:
            side.forward(ctx, x, xr if wants_rounded else x)
