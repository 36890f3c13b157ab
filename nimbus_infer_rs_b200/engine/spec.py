"""The description of a model as data: which parts, layer by layer, and in which order.

An architecture's ``build_spec(config)`` returns a :class:`ModelSpec`; the engine builds the
model from it without knowing the architecture.  Layers may differ from one another
(another mixer, another feed-forward), ``schedule`` lists the layers in the order they run
(a layer may be named twice: it then runs with the same parameters and a cache or state of
its own each time), and a layer with ``cache_from`` set reads the key/value cache of that
other layer instead of keeping its own.  A layer may have no feed-forward (``ffn=None``), and
an arrangement in which both sublayers read one norm has no second norm (``norm_ffn=None``).
``max_seq_len=None``: nothing in the model bounds a sequence; the cache's size does.
``stream_input`` with ``stream_input_before``: a part of the ``stream`` family (one set of
parameters) that transforms the stream right before each of the named schedule entries, from
the stream and the embedding's output.  ``logit_scale`` multiplies the logits.  ``embedding``: a
part of the ``embedding`` family in place of the plain token table.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..parts.base import PartSpec


@dataclass(frozen=True)
class LayerSpec:
    mixer: PartSpec
    ffn: PartSpec | None
    norm_mixer: PartSpec
    norm_ffn: PartSpec | None
    block: PartSpec = PartSpec("pre_norm")
    cache_from: int | None = None
    # norms of the sublayers' results, for an arrangement that has them (``sandwich``)
    post_norm_mixer: PartSpec | None = None
    post_norm_ffn: PartSpec | None = None
    # a per-token input added to the stream after the sublayers
    side: PartSpec | None = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    width: int
    max_seq_len: int | None
    position: PartSpec
    layers: tuple[LayerSpec, ...]
    final_norm: PartSpec
    tie_head: bool = True
    schedule: tuple[int, ...] | None = None
    embedding_scale: float = 1.0      # multiplies the token embedding (not the tied head)
    logit_scale: float = 1.0          # multiplies the logits
    # another way from tokens to the stream than the token table (``embedding`` family); its
    # arguments must include ``vocab_size`` and ``width``
    embedding: PartSpec | None = None
    stream_input: PartSpec | None = None
    stream_input_before: tuple[int, ...] = ()     # schedule entries (positions in the run order)

    def run_order(self) -> tuple[int, ...]:
        order = self.schedule if self.schedule is not None else tuple(range(len(self.layers)))
        for i in order:
            if not 0 <= i < len(self.layers):
                raise ValueError(f"schedule names layer {i}, but there are {len(self.layers)}")
        return tuple(order)

    def validate(self) -> None:
        n_entries = len(self.run_order())
        if self.stream_input_before and self.stream_input is None:
            raise ValueError("stream_input_before names entries, but there is no stream_input")
        for e in self.stream_input_before:
            if not 0 <= e < n_entries:
                raise ValueError(f"stream_input_before names entry {e} of {n_entries}")
        for i, l in enumerate(self.layers):
            if l.cache_from is not None:
                if not 0 <= l.cache_from < len(self.layers) or l.cache_from == i:
                    raise ValueError(f"layer {i}: cache_from={l.cache_from} is not another layer")
                if self.layers[l.cache_from].cache_from is not None:
                    raise ValueError(f"layer {i}: cache_from must name a layer with its own cache")
