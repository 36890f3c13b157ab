"""Lulizen as data: how its configuration maps onto parts, and where its parameters are found in
a weight file.  This is the only file that knows the architecture.

Structure: the token's embedding plus a row of a second table picked by a hash of the token and
the one before it; layers in any order of two kinds of attention, ``attention`` (queries and
keys normed per head, a mask by blocks of positions, a sink) and ``attention_2`` (a sliding
window that also keeps the sequence's first tokens, a gate per head), both with rotated queries
and keys and capped scores; every sublayer between two layer norms (a weight, no shift), its
normed result added to the stream; a feed-forward per layer that is dense and gated (tanh
gelu), routed experts chosen by sigmoid scores among the best groups (plus a shared expert), or
absent; a final layer norm and an output head of its own.  A layer may run with another
layer's tensors and a cache of its own.

Tensor names: ``embed``, ``bigram``, ``final.norm``, ``head``, and per layer ``l<i>.``:
``norm1``, ``norm1b``, ``norm2``, ``norm2b``, ``mix.{q, k, v, o}`` with ``mix.{q.norm, k.norm,
sink}`` or ``mix.g``, ``mlp.{gate, up, down}`` or ``mlp.{router, correction, e<k>.{gate, up,
down}, shared.{gate, up, down}}``; every linear weight stored ``(out, in)``.
"""
from __future__ import annotations

import math

import torch

from ..config.lulizen import GROUP_TOP, DenseFFConfig, LulizenConfig, MoEFFConfig
from ..config.registry import Architecture, register_architecture
from ..engine.spec import LayerSpec, ModelSpec
from ..parts.base import PartSpec
from ..weights.loader import Recipe, WeightPlan, take
from .runesun import _rows, _stack

NORM_SUM_EPS = 1e-20      # joins the sum of the chosen experts' scores before the division


def _owners(cfg: LulizenConfig) -> list[int]:
    """The layers that have tensors of their own, in order."""
    return [i for i, l in enumerate(cfg.layers) if l.weights_of is None]


def _limit(e) -> float | None:
    return e.limit


def _ffn_spec(D: int, ff) -> PartSpec | None:
    if ff is None:
        return None
    if isinstance(ff, DenseFFConfig):
        return PartSpec("gated_mlp", {"width": D, "hidden": ff.ff, "activation": "gelu_tanh"})
    shared = None if ff.shared is None else {
        "hidden": ff.shared.ff, "activation": "swish_clamp", "limit": ff.shared.limit}
    return PartSpec("routed_experts", {
        "width": D, "n_experts": ff.experts, "top": ff.top, "hidden": ff.expert.ff,
        "activation": "swish_clamp", "limit": ff.expert.limit, "gated": True,
        "scores": "sigmoid", "correction": ff.correction, "groups": ff.groups,
        "keep_groups": ff.keep_groups, "group_top": GROUP_TOP, "renormalize": True,
        "norm_eps": NORM_SUM_EPS, "route_scale": ff.route_scale, "shared": shared})


def build_spec(cfg: LulizenConfig) -> ModelSpec:
    D = cfg.width
    norm = PartSpec("layernorm", {"width": D, "eps": cfg.norm_eps, "bias": False})
    owners = _owners(cfg)
    layers = []
    for i in owners:
        l = cfg.layers[i]
        mx = l.mixer
        blocks = l.type == "attention"
        mixer = PartSpec("masked_attention", {
            "width": D, "n_heads": mx.heads, "n_kv_heads": mx.kv_heads, "head_dim": mx.dim,
            "value_dim": mx.vdim, "scale": mx.scale, "eps": cfg.norm_eps, "qk_norm": blocks,
            "softcap": mx.softcap, "window": 0 if blocks else mx.mask_size,
            "keep_first": 0 if blocks else mx.keep_first, "chunk": mx.mask_size if blocks else 0,
            "sink": blocks, "gate": not blocks,
            "rot_dims": 0 if mx.rot is None else mx.rot.dims,
            "rot_base": 10000.0 if mx.rot is None else mx.rot.base})
        ffn = _ffn_spec(D, l.mlp)
        layers.append(LayerSpec(
            mixer=mixer, ffn=ffn, norm_mixer=norm, norm_ffn=None if ffn is None else norm,
            block=PartSpec("sandwich"), post_norm_mixer=norm,
            post_norm_ffn=None if ffn is None else norm))
    embedding = None if cfg.bigram is None else PartSpec("hashed_pair_embedding", {
        "vocab_size": cfg.vocab_size, "width": D, "buckets": cfg.bigram.buckets,
        "mul_prev": cfg.bigram.mul_prev, "mul_cur": cfg.bigram.mul_cur})
    return ModelSpec(
        architecture="lulizen", vocab_size=cfg.vocab_size, width=D, max_seq_len=None,
        position=PartSpec("none"), layers=tuple(layers), final_norm=norm, tie_head=False,
        schedule=tuple(owners.index(cfg.owner(i)) for i in range(len(cfg.layers))),
        embedding=embedding)


def weight_plan(cfg: LulizenConfig, spec: ModelSpec, names: set[str]) -> WeightPlan:
    D, V = cfg.width, cfg.vocab_size
    r: dict[str, Recipe] = {"embedding.table": take("embed", (V, D)),
                            "final_norm.weight": take("final.norm", (D,)),
                            "head.weight": take("head", (V, D))}
    if cfg.bigram is not None:
        r["embedding.pair_table"] = take("bigram", (cfg.bigram.buckets + 1, D))
    ignored = set()
    for n, i in enumerate(_owners(cfg)):
        l = cfg.layers[i]
        mx, ff = l.mixer, l.mlp
        H, G, d, dv = mx.heads, mx.kv_heads, mx.dim, mx.vdim
        p, L = f"l{i}.", f"layers.{n}."
        r[L + "norm_mixer.weight"] = take(p + "norm1", (D,))
        r[L + "post_norm_mixer.weight"] = take(p + "norm1b", (D,))
        fused = [(p + "mix.q", (H * d, D)), (p + "mix.k", (G * d, D)), (p + "mix.v", (G * dv, D))]
        if l.type == "attention":
            r[L + "mixer.q_norm"] = take(p + "mix.q.norm", (d,))
            r[L + "mixer.k_norm"] = take(p + "mix.k.norm", (d,))
            r[L + "mixer.sink"] = take(p + "mix.sink", (H,))
        else:
            fused.append((p + "mix.g", (H, D)))
        r[L + "mixer.proj.weight"] = _rows(fused, multiple=8)
        r[L + "mixer.out.weight"] = take(p + "mix.o", (D, H * dv))
        if ff is None:
            # a layer without a feed-forward may still carry the norms around it in the file
            ignored |= {p + "norm2", p + "norm2b"}
            continue
        r[L + "norm_ffn.weight"] = take(p + "norm2", (D,))
        r[L + "post_norm_ffn.weight"] = take(p + "norm2b", (D,))
        if isinstance(ff, DenseFFConfig):
            r[L + "ffn.fc.weight"] = _gate_up(p + "mlp.", ff.ff, D)
            r[L + "ffn.proj.weight"] = take(p + "mlp.down", (D, ff.ff))
        else:
            E, F = ff.experts, ff.expert.ff
            if ff.shared is None:
                r[L + "ffn.router.weight"] = take(p + "mlp.router", (E, D))
            if ff.correction:
                r[L + "ffn.correction"] = take(p + "mlp.correction", (E,))
            r[L + "ffn.gate"] = _stack([f"{p}mlp.e{k}.gate" for k in range(E)], (F, D))
            r[L + "ffn.up"] = _stack([f"{p}mlp.e{k}.up" for k in range(E)], (F, D))
            r[L + "ffn.down"] = _stack([f"{p}mlp.e{k}.down" for k in range(E)], (D, F))
            if ff.shared is not None:
                # the router's rows ride under the shared expert's gate and up halves
                r[L + "ffn.shared.fc.weight"] = _gate_up(p + "mlp.shared.", ff.shared.ff, D,
                                                         extra=(p + "mlp.router", E))
                r[L + "ffn.shared.proj.weight"] = take(p + "mlp.shared.down", (D, ff.shared.ff))
    return WeightPlan(r, ignored)


def _gate_up(prefix: str, hidden: int, width: int, extra: tuple[str, int] | None = None) -> Recipe:
    """Gate and up one under the other, each half filled with rows of zeros up to a multiple of
    8 rows (the layout of ``gated_mlp``'s first product); ``extra`` = (name, rows): one more
    matrix under them, filled up likewise."""
    named = [(prefix + "gate", (hidden, width)), (prefix + "up", (hidden, width))]
    if extra is not None:
        named.append((extra[0], (extra[1], width)))
    inner = _rows(named)

    def combine(ts):
        kinds = {t.dtype for t in ts}
        if len(kinds) > 1:
            ts = [t.to(torch.float32) for t in ts]
        out = []
        for t in ts:
            out.append(t)
            pad = -t.shape[0] % 8
            if pad:
                out.append(torch.zeros((pad, width), dtype=t.dtype))
        return torch.cat(out, dim=0).contiguous()
    return Recipe(inner.sources, combine)


def complete_config(cfg: LulizenConfig, shapes: dict) -> LulizenConfig:
    return cfg.with_shapes(shapes)


def random_tensors(cfg: LulizenConfig, seed: int, *, gain: float = 1.0, std: float | None = None,
                   sink_std: float = 1.0, gamma_jitter: float = 0.1, correction_std: float = 0.1,
                   dtype: torch.dtype = torch.bfloat16) -> dict:
    """Random Lulizen tensors under the names of a weight file.  Matrices ~N(0, gain^2 / in) (or
    ~N(0, std^2) if ``std`` is given), embeddings ~N(0, 1), norm weights 1 + N(0, gamma_jitter^2),
    sinks ~N(0, sink_std^2), choice biases ~N(0, correction_std^2); drawn in fp32 from a seeded
    CPU generator in a fixed order and stored in ``dtype``."""
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))

    def mat(n_out, n_in, s=None):
        s = (gain / math.sqrt(n_in) if std is None else std) if s is None else s
        return (torch.randn(n_out, n_in, generator=g, dtype=torch.float32) * s).to(dtype)

    def vec(n, s, mean=0.0):
        return (torch.randn(n, generator=g, dtype=torch.float32) * s + mean).to(dtype)

    def expert(p, hidden):
        out[p + "gate"] = mat(hidden, D)
        out[p + "up"] = mat(hidden, D)
        out[p + "down"] = mat(D, hidden)

    D, V = cfg.width, cfg.vocab_size
    out: dict[str, torch.Tensor] = {"embed": mat(V, D, 1.0)}
    if cfg.bigram is not None:
        out["bigram"] = mat(cfg.bigram.buckets + 1, D, 0.5)
    for i in _owners(cfg):
        l = cfg.layers[i]
        mx, ff = l.mixer, l.mlp
        H, G, d, dv = mx.heads, mx.kv_heads, mx.dim, mx.vdim
        p = f"l{i}."
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if ff is not None else ()):
            out[p + n] = vec(D, gamma_jitter, 1.0)
        out[p + "mix.q"] = mat(H * d, D)
        out[p + "mix.k"] = mat(G * d, D)
        out[p + "mix.v"] = mat(G * dv, D)
        if l.type == "attention":
            out[p + "mix.q.norm"] = vec(d, gamma_jitter, 1.0)
            out[p + "mix.k.norm"] = vec(d, gamma_jitter, 1.0)
            out[p + "mix.sink"] = vec(H, sink_std)
        else:
            out[p + "mix.g"] = mat(H, D)
        out[p + "mix.o"] = mat(D, H * dv)
        if isinstance(ff, DenseFFConfig):
            expert(p + "mlp.", ff.ff)
        elif isinstance(ff, MoEFFConfig):
            for k in range(ff.experts):
                expert(f"{p}mlp.e{k}.", ff.expert.ff)
            out[p + "mlp.router"] = mat(ff.experts, D)
            if ff.correction:
                out[p + "mlp.correction"] = vec(ff.experts, correction_std)
            if ff.shared is not None:
                expert(p + "mlp.shared.", ff.shared.ff)
    out["final.norm"] = vec(D, gamma_jitter, 1.0)
    out["head"] = mat(V, D)
    return out


ARCHITECTURE = register_architecture(Architecture(
    name="lulizen", config_cls=LulizenConfig, build_spec=build_spec, weight_plan=weight_plan,
    aliases=("Lulizen",), random_tensors=random_tensors, complete_config=complete_config),
    replace=True)
