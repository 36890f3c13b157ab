"""Typed configuration of the Lulizen decoder.

config.json of this design::

    {"architecture": "Lulizen", "vocab": V, "width": D, "norm": {"eps": e},
     "embedding": {"bigram": {"buckets": B, "mul_prev": a, "mul_cur": b}},
     "layers": [
       {"type": "attention",
        "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": c, "softcap": s,
                  "rot": {"dims": r, "base": b}, "mask": {"size": C}},
        "mlp": {"kind": "dense", "ff": F}
             | {"kind": "moe", "expert": {"ff": F, "limit": L},
                "router": {"experts": E, "top": k, "scale": w,
                           "groups": {"count": n, "keep": m}},
                "shared": {"ff": Fs, "limit": Ls}}
             | null,
        "weights_of": j (optional)},
       {"type": "attention_2",
        "mixer": {... as above ..., "mask": {"size": W, "keep_first": K}}, "mlp": ...}, ...]}

Every size and constant is read from there; layers come in any order and may differ from one
another.  ``attention`` norms queries and keys per head, sees the tokens of its own block of
``mask.size`` positions and has a sink; ``attention_2`` sees a sliding window of ``mask.size``
tokens plus the sequence's first ``mask.keep_first`` and gates every head's result.  Optional
keys: ``embedding.bigram`` (no second table), ``kv_heads`` (= heads), ``vdim`` (= dim),
``softcap`` (none), ``rot`` (no rotation), ``mask`` (every earlier token), ``mask.keep_first``
(0), ``router.scale`` (1), ``router.groups`` (no groups), ``shared`` (no shared expert),
``limit`` (no bound), ``router.correction: false`` (no choice bias).  A layer with ``weights_of: j`` has no tensors of its own and runs with
layer ``j``'s (its own cache).  Whether a router has a choice bias is read off the weight
file (``complete_config``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Any

from .base import ConfigError
from .runesun import _float, _int

MIXER_TYPES = ("attention", "attention_2")
MLP_KINDS = ("dense", "moe")
GROUP_TOP = 2            # a group's score is the sum of this many of its best choice scores


@dataclass(frozen=True)
class RotaryConfig:
    dims: int
    base: float


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float = 0.0          # 0: scores are not capped
    rot: RotaryConfig | None = None
    mask_size: int = 0            # 0: every earlier token is seen
    keep_first: int = 0           # attention_2: first tokens seen beside the window


@dataclass(frozen=True)
class DenseFFConfig:
    ff: int


@dataclass(frozen=True)
class ExpertConfig:
    ff: int
    limit: float                  # inf: no bound


@dataclass(frozen=True)
class MoEFFConfig:
    experts: int
    top: int
    expert: ExpertConfig
    route_scale: float = 1.0
    groups: int = 1
    keep_groups: int = 1
    shared: ExpertConfig | None = None
    correction: bool = True       # the router has a choice bias (off if the weight file has none)


@dataclass(frozen=True)
class LulizenLayerConfig:
    type: str
    mixer: AttentionConfig
    mlp: Any                      # DenseFFConfig, MoEFFConfig or None
    weights_of: int | None = None


@dataclass(frozen=True)
class BigramConfig:
    buckets: int
    mul_prev: int
    mul_cur: int


def _limit(problems, where, obj) -> float:
    if not isinstance(obj, dict) or obj.get("limit") is None:
        return math.inf
    return _float(problems, where, obj, "limit")


def _read_mixer(problems, where, kind, m) -> AttentionConfig:
    has = (lambda k: isinstance(m, dict) and m.get(k) is not None)
    heads = _int(problems, where, m, "heads")
    kv_heads = _int(problems, where, m, "kv_heads") if has("kv_heads") else heads
    dim = _int(problems, where, m, "dim")
    vdim = _int(problems, where, m, "vdim") if has("vdim") else dim
    if heads % kv_heads:
        problems.append(f"{where}: heads={heads} is no multiple of kv_heads={kv_heads}")
    scale = _float(problems, where, m, "scale", positive=False) if has("scale") else dim ** -0.5
    softcap = _float(problems, where, m, "softcap") if has("softcap") else 0.0
    rot = None
    if has("rot"):
        r = m["rot"]
        dims = _int(problems, where + ".rot", r, "dims", minimum=2)
        if dims % 2 or dims > dim:
            problems.append(f"{where}.rot.dims: {dims} must be even and at most the head's {dim}")
        rot = RotaryConfig(dims, _float(problems, where + ".rot", r, "base"))
    size = keep = 0
    if has("mask"):
        mask = m["mask"]
        size = _int(problems, where + ".mask", mask, "size")
        if isinstance(mask, dict) and mask.get("keep_first") is not None:
            keep = _int(problems, where + ".mask", mask, "keep_first", minimum=0)
            if kind != "attention_2":
                problems.append(f"{where}.mask.keep_first: only a sliding window keeps first tokens")
    return AttentionConfig(heads, kv_heads, dim, vdim, scale, softcap, rot, size, keep)


def _read_mlp(problems, where, f):
    if f is None:
        return None
    if not isinstance(f, dict) or f.get("kind") not in MLP_KINDS:
        problems.append(f"{where}.kind: unknown feed-forward "
                        f"{f.get('kind') if isinstance(f, dict) else f!r} "
                        f"(known: {list(MLP_KINDS)}, or null)")
        return None
    if f["kind"] == "dense":
        return DenseFFConfig(ff=_int(problems, where, f, "ff"))
    r, e = f.get("router"), f.get("expert")
    experts = _int(problems, where + ".router", r, "experts")
    top = _int(problems, where + ".router", r, "top")
    if top > experts:
        problems.append(f"{where}.router: top={top} of {experts} experts")
    route_scale = 1.0
    if isinstance(r, dict) and r.get("scale") is not None:
        route_scale = _float(problems, where + ".router", r, "scale", positive=False)
    groups = keep = 1
    if isinstance(r, dict) and r.get("groups") is not None:
        g = r["groups"]
        groups = _int(problems, where + ".router.groups", g, "count")
        keep = _int(problems, where + ".router.groups", g, "keep")
        if experts % groups or keep > groups or keep * (experts // max(groups, 1)) < top:
            problems.append(f"{where}.router.groups: {groups} groups (keep {keep}) do not fit "
                            f"{experts} experts with top={top}")
    shared = None
    if f.get("shared") is not None:
        s = f["shared"]
        shared = ExpertConfig(_int(problems, where + ".shared", s, "ff"),
                              _limit(problems, where + ".shared", s))
    correction = not (isinstance(r, dict) and r.get("correction") is False)
    return MoEFFConfig(experts=experts, top=top, correction=correction,
                       expert=ExpertConfig(_int(problems, where + ".expert", e, "ff"),
                                           _limit(problems, where + ".expert", e)),
                       route_scale=route_scale, groups=groups, keep_groups=keep, shared=shared)


@dataclass(frozen=True)
class LulizenConfig:
    architecture = "lulizen"

    vocab_size: int
    width: int
    norm_eps: float
    bigram: BigramConfig | None
    layers: tuple[LulizenLayerConfig, ...]
    name: str = "model"

    @classmethod
    def from_json(cls, obj: dict) -> "LulizenConfig":
        if not isinstance(obj, dict):
            raise ConfigError("config.json must hold a JSON object")
        problems: list[str] = []
        vocab = _int(problems, "config", obj, "vocab")
        width = _int(problems, "config", obj, "width")
        eps = _float(problems, "norm", obj.get("norm"), "eps")
        bigram = None
        emb = obj.get("embedding")
        if isinstance(emb, dict) and emb.get("bigram") is not None:
            b = emb["bigram"]
            bigram = BigramConfig(_int(problems, "embedding.bigram", b, "buckets"),
                                  _int(problems, "embedding.bigram", b, "mul_prev", minimum=0),
                                  _int(problems, "embedding.bigram", b, "mul_cur", minimum=0))
        raw_layers = obj.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("bad config.json: layers: expected a non-empty list"
                              + ("; " + "; ".join(problems) if problems else ""))
        layers = []
        for i, entry in enumerate(raw_layers):
            where = f"layers[{i}]"
            if not isinstance(entry, dict):
                problems.append(f"{where}: expected an object")
                continue
            kind = entry.get("type")
            if kind not in MIXER_TYPES:
                problems.append(f"{where}.type: unknown mixer {kind!r} (known: {list(MIXER_TYPES)})")
                continue
            mixer = _read_mixer(problems, where + ".mixer", kind, entry.get("mixer"))
            mlp = _read_mlp(problems, where + ".mlp", entry.get("mlp"))
            wo = entry.get("weights_of")
            if wo is not None:
                if isinstance(wo, bool) or not isinstance(wo, int) or not 0 <= wo < len(raw_layers) \
                        or wo == i:
                    problems.append(f"{where}.weights_of: {wo!r} is not another layer")
                    wo = None
            layers.append(LulizenLayerConfig(kind, mixer, mlp, wo))
        if problems:
            raise ConfigError("bad config.json: " + "; ".join(problems))
        cfg = cls(vocab_size=vocab, width=width, norm_eps=eps, bigram=bigram, layers=tuple(layers),
                  name=str(obj.get("name", "model")))
        for i, l in enumerate(layers):
            j = cfg.owner(i)              # a chain that never reaches tensors fails here
            o = layers[j]
            if j != i and (o.type, o.mixer, o.mlp) != (l.type, l.mixer, l.mlp):
                raise ConfigError(f"bad config.json: layers[{i}] runs with the tensors of layer {j} "
                                  "but is described differently")
        return cfg

    def owner(self, i: int) -> int:
        """The layer whose tensors layer ``i`` runs with (``i`` itself if it has its own)."""
        seen = set()
        while self.layers[i].weights_of is not None:
            if i in seen:
                raise ConfigError(f"bad config.json: layers[{i}].weights_of goes round in a circle")
            seen.add(i)
            i = self.layers[i].weights_of
        return i

    def with_shapes(self, shapes: dict) -> "LulizenConfig":
        """What only the weight file tells: whether a router comes with a choice bias."""
        layers = []
        for i, l in enumerate(self.layers):
            if isinstance(l.mlp, MoEFFConfig):
                has = f"l{self.owner(i)}.mlp.correction" in shapes
                l = replace(l, mlp=replace(l.mlp, correction=has and l.mlp.correction))
            layers.append(l)
        return replace(self, layers=tuple(layers))

    def n_params(self, *_unused) -> int:
        D = self.width
        total = 2 * self.vocab_size * D + D
        if self.bigram is not None:
            total += (self.bigram.buckets + 1) * D
        for l in self.layers:
            if l.weights_of is not None:
                continue
            m = l.mixer
            total += (4 if l.mlp is not None else 2) * D
            total += (m.heads * m.dim + m.kv_heads * (m.dim + m.vdim)) * D + m.heads * m.vdim * D
            total += 2 * m.dim + m.heads if l.type == "attention" else m.heads * D
            if isinstance(l.mlp, DenseFFConfig):
                total += 3 * l.mlp.ff * D
            elif isinstance(l.mlp, MoEFFConfig):
                total += l.mlp.experts * (3 * l.mlp.expert.ff * D + D)
                total += l.mlp.experts if l.mlp.correction else 0
                if l.mlp.shared is not None:
                    total += 3 * l.mlp.shared.ff * D
        return total

    def to_json(self) -> dict[str, Any]:
        def expert(e: ExpertConfig) -> dict:
            return {"ff": e.ff, **({} if math.isinf(e.limit) else {"limit": e.limit})}

        out = []
        for l in self.layers:
            m = l.mixer
            mx: dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim,
                                  "vdim": m.vdim, "scale": m.scale}
            if m.softcap:
                mx["softcap"] = m.softcap
            if m.rot is not None:
                mx["rot"] = {"dims": m.rot.dims, "base": m.rot.base}
            if m.mask_size:
                mx["mask"] = {"size": m.mask_size,
                              **({"keep_first": m.keep_first} if l.type == "attention_2" else {})}
            if l.mlp is None:
                ff = None
            elif isinstance(l.mlp, DenseFFConfig):
                ff = {"kind": "dense", "ff": l.mlp.ff}
            else:
                f = l.mlp
                router: dict[str, Any] = {"experts": f.experts, "top": f.top, "scale": f.route_scale}
                if not f.correction:
                    router["correction"] = False
                if f.groups > 1:
                    router["groups"] = {"count": f.groups, "keep": f.keep_groups}
                ff = {"kind": "moe", "expert": expert(f.expert), "router": router}
                if f.shared is not None:
                    ff["shared"] = expert(f.shared)
            e: dict[str, Any] = {"type": l.type, "mixer": mx, "mlp": ff}
            if l.weights_of is not None:
                e["weights_of"] = l.weights_of
            out.append(e)
        obj: dict[str, Any] = {"architecture": "Lulizen", "name": self.name, "vocab": self.vocab_size,
                               "width": self.width, "norm": {"eps": self.norm_eps}, "layers": out}
        if self.bigram is not None:
            obj["embedding"] = {"bigram": {"buckets": self.bigram.buckets,
                                           "mul_prev": self.bigram.mul_prev,
                                           "mul_cur": self.bigram.mul_cur}}
        return obj
