"""A model assembled from a :class:`ModelSpec`: embedding, position encoding, layers in
schedule order, final norm, output head.  It owns no architecture knowledge.

The forward pass follows src/model.rs:271-325: embed (+ position), every scheduled layer on
the fp32 residual stream, then the final norm and the head -- here only on the rows whose
logits were asked for (the reference norms every row and takes logits of the last one).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import ParamSpec, bind_params, build_part, collect_param_specs
from ..parts.embedding import LMHead, TokenEmbedding
from .spec import ModelSpec

EMBEDDING_ENTRY = -1     # the key of the embedding's state rows among the schedule entries

PRECISIONS = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
              "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


@dataclass
class Runtime:
    """What every part may ask about the run: device and element type of activations and
    caches (``bfloat16``: the serving precision; ``float32``: everything in true 32-bit)."""
    device: torch.device
    act_dtype: torch.dtype

    @property
    def precision(self) -> str:
        return "float32" if self.act_dtype == torch.float32 else "bfloat16"


class Layer:
    def __init__(self, index: int, spec):
        self.index = index
        self.spec = spec
        self.block = build_part("block", spec.block)
        self.norm_mixer = build_part("norm", spec.norm_mixer)
        self.mixer = build_part("mixer", spec.mixer)
        self.norm_ffn = build_part("norm", spec.norm_ffn) if spec.norm_ffn is not None else None
        self.ffn = build_part("ffn", spec.ffn) if spec.ffn is not None else None
        self.post_norm_mixer = build_part("norm", spec.post_norm_mixer) \
            if spec.post_norm_mixer is not None else None
        self.post_norm_ffn = build_part("norm", spec.post_norm_ffn) \
            if spec.post_norm_ffn is not None else None
        self.side = build_part("side", spec.side) if spec.side is not None else None

    def parts(self):
        """The layer's parts that exist, by the name their parameters are listed under."""
        named = {"norm_mixer": self.norm_mixer, "mixer": self.mixer,
                 "norm_ffn": self.norm_ffn, "ffn": self.ffn,
                 "post_norm_mixer": self.post_norm_mixer, "post_norm_ffn": self.post_norm_ffn,
                 "side": self.side}
        return {k: v for k, v in named.items() if v is not None}


class Model:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        spec.validate()
        self.spec = spec
        self.rt = runtime
        self.embedding = TokenEmbedding(spec.vocab_size, spec.width, spec.embedding_scale) \
            if spec.embedding is None else build_part("embedding", spec.embedding)
        self.position = build_part("position", spec.position)
        self.layers = [Layer(i, ls) for i, ls in enumerate(spec.layers)]
        final_norm = spec.final_norm
        if spec.logit_scale != 1.0:
            # logits = head(norm(x)) * c = head(c * norm(x)): the constant rides on the norm
            final_norm = final_norm.with_args(gain=spec.logit_scale)
        self.final_norm = build_part("norm", final_norm)
        self.stream_input = build_part("stream", spec.stream_input) \
            if spec.stream_input is not None else None
        self.stream_input_before = frozenset(spec.stream_input_before)
        self.head = LMHead(spec.vocab_size, spec.width, spec.tie_head)
        self.run_order = spec.run_order()
        self.params: dict[str, torch.Tensor | None] = {}

    # ------------------------------------------------------------------ parameters
    def _named_parts(self):
        yield "embedding.", self.embedding
        yield "position.", self.position
        for l in self.layers:
            for name, part in l.parts().items():
                yield f"layers.{l.index}.{name}.", part
        if self.stream_input is not None:
            yield "stream_input.", self.stream_input
        yield "final_norm.", self.final_norm
        yield "head.", self.head

    def param_specs(self) -> dict[str, ParamSpec]:
        out: dict[str, ParamSpec] = {}
        for prefix, part in self._named_parts():
            out.update(collect_param_specs(part, prefix))
        return out

    def bind(self, params: dict[str, torch.Tensor | None]) -> None:
        self.params = params
        for prefix, part in self._named_parts():
            bind_params(part, params, self.rt, prefix)
        if self.spec.tie_head:
            self.head.tie(self.embedding.table)

    def graph_safe(self) -> bool:
        """True if every part of the model may run under CUDA-graph capture."""
        parts = [self.embedding, self.position, self.final_norm, self.head]
        if self.stream_input is not None:
            parts.append(self.stream_input)
        for l in self.layers:
            parts += [l.block, *l.parts().values()]
        return all(getattr(p, "graph_safe", False) for p in parts)

    def n_params(self) -> int:
        return sum(t.numel() for t in self.params.values() if t is not None)

    def weight_bytes(self) -> int:
        """Bytes of the tensors a decode step reads: every parameter once, except that of the
        embedding tables only the rows of the step's tokens are read (the tied table is
        counted because the head reads all of it)."""
        total = 0
        for name, t in self.params.items():
            if t is None:
                continue
            if name == "position.table" or (name == "embedding.table" and not self.spec.tie_head):
                continue
            total += t.numel() * t.element_size()
        return total

    # ------------------------------------------------------------------ forward
    def forward_hidden(self, ctx) -> torch.Tensor:
        """The fp32 residual stream after the last scheduled layer, [rows, width]."""
        ctx.state = ctx.cache.layer_state(EMBEDDING_ENTRY)
        x = self.embedding.forward(ctx, self.position)
        x0 = x
        if self.stream_input_before and min(self.stream_input_before) > 0:
            # the layers add into the stream in place: the embedding's output is kept apart
            x = torch.empty_like(x0)
            ctx.ops.cast_cols(x0, x, 0)
        for entry, li in enumerate(self.run_order):
            layer = self.layers[li]
            if entry in self.stream_input_before:
                x = self.stream_input.forward(ctx, x, x0)
                ctx.normed = None
            ctx.kv, ctx.state, ctx.writes_cache = self.storage_of(ctx.cache, entry)
            ctx.kv_extra = ctx.cache.layer_kv_extra(entry)
            # an arrangement whose last pass over the stream can also norm it for the entry that
            # runs next is told that entry's first norm
            ctx.next_norm = None
            if entry + 1 < len(self.run_order) and entry + 1 not in self.stream_input_before:
                nxt = self.layers[self.run_order[entry + 1]]
                if getattr(nxt.block, "takes_handed_norm", False):
                    ctx.next_norm = nxt.norm_mixer
            layer.block.forward(ctx, x, layer)
        ctx.next_norm = ctx.normed = None
        return x

    def storage_requests(self):
        """What each schedule entry keeps per sequence: ``({entry: KVRequest}, {entry:
        StateRequest})``.  An entry of a layer with ``cache_from`` keeps no keys/values."""
        kv, st = {}, {}
        for entry, li in enumerate(self.run_order):
            layer = self.layers[li]
            r = layer.mixer.cache_request()
            if layer.spec.cache_from is None:
                if r is not None:
                    kv[entry] = r
            else:
                # the reader must want what the owner keeps: same heads and head size, and no
                # keys from before the owner's window
                own = self.layers[layer.spec.cache_from].mixer.cache_request()
                ok = (r is not None and own is not None and r.n_kv_heads == own.n_kv_heads
                      and r.head_dim == own.head_dim
                      and (own.window == 0 or 0 < r.window <= own.window))
                if not ok:
                    raise ValueError(
                        f"layer {li} reads the cache of layer {layer.spec.cache_from}, which "
                        f"keeps {own}, but asks for {r}")
            s = layer.mixer.state_request()
            if s is not None:
                st[entry] = s
        s = self.embedding.state_request()
        if s is not None:
            st[EMBEDDING_ENTRY] = s
        return kv, st

    def extra_storage_requests(self):
        """The further paged stores of each schedule entry's mixer: ``{(entry, k): KVRequest}``."""
        out = {}
        for entry, li in enumerate(self.run_order):
            for k, r in enumerate(self.layers[li].mixer.extra_cache_requests()):
                out[(entry, k)] = r
        return out

    def kv_source(self, entry: int) -> int:
        """The schedule entry whose key/value store ``entry`` uses: itself, or the latest
        earlier run of the layer named by ``cache_from``."""
        src = self.layers[self.run_order[entry]].spec.cache_from
        if src is None:
            return entry
        for e in range(entry - 1, -1, -1):
            if self.run_order[e] == src:
                return e
        raise ValueError(f"schedule entry {entry}: layer {src}, whose cache it reads, has not "
                         "run before it")

    def storage_of(self, cache, entry: int):
        src = self.kv_source(entry)
        return cache.layer_kv(src), cache.layer_state(entry), src == entry

    def logits(self, ctx, x: torch.Tensor, rows: torch.Tensor, n_rows: int) -> torch.Tensor:
        """Final norm and head on the selected rows → fp32 [n_rows, vocab]."""
        if ctx.layout.want_all_rows and n_rows == x.shape[0]:
            # every row is wanted, in order (a decode step): no gather, and the norm may be
            # folded into the head's product
            return self.head.forward(ctx, self.final_norm.defer(ctx, x))
        h = self.final_norm.forward(ctx, x, rows, n_rows)
        return self.head.forward(ctx, h)

    def forward(self, ctx) -> torch.Tensor | None:
        x = self.forward_hidden(ctx)
        lay = ctx.layout
        if lay.n_want == 0:
            return None
        return self.logits(ctx, x, lay.want_rows, lay.n_want)
