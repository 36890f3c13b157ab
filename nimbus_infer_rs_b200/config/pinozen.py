"""Typed configuration of the Pinozen decoder.

config.json of this design::

    {"architecture": "Pinozen", "vocab": V, "width": D, "max_positions": P,
     "norm": {"eps": e}, "embedding": {"scale": s}, "logit_scale": c,
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [
       {"type": "parallel",
        "mixer": {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "conv": taps,
                           "scale": c, "softcap": cap,
                           "rot": {"dims": r, "base": b,
                                   "scaling": {"factor": f, "low": x, "high": y, "original": n}}},
                  "right": {"inner": I, "state": N, "dt_rank": R, "conv": taps}},
        "mlp": {"kind": "dense", "ff": F} | null},
       {"type": "lightning",
        "mixer": {"heads": H, "dim": d, "vdim": dv, "decay": [w_0, ..., w_(H-1)]},
        "mlp": ...}, ...]}

Every size and constant is read from there; layers come in any order and may differ from one
another.  Left out means absent: no ``loop`` (every layer runs once), no ``embedding`` or
``logit_scale`` (a factor of one), no ``kv_heads`` (as many as heads), no ``vdim`` (``dim``), no
``conv`` (no convolution), no ``softcap``, no ``rot`` (no rotation), no ``rot.scaling``.  Without
``max_positions`` the position table's size comes from the weight file's shapes.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any

from .base import ConfigError
from .runesun import _float, _int

MIXER_TYPES = ("parallel", "lightning")
MLP_KINDS = ("dense",)


@dataclass(frozen=True)
class WavelengthScaling:
    factor: float
    low: float
    high: float
    original: float


@dataclass(frozen=True)
class PairedRotaryConfig:
    dims: int
    base: float
    scaling: WavelengthScaling | None = None


@dataclass(frozen=True)
class CappedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int = 0              # taps of the short convolution; 0: none
    softcap: float = 0.0       # 0: scores are not capped
    rot: PairedRotaryConfig | None = None


@dataclass(frozen=True)
class ScanConfig:
    inner: int
    state: int
    dt_rank: int
    conv: int = 0


@dataclass(frozen=True)
class PairMixerConfig:
    left: CappedAttentionConfig
    right: ScanConfig


@dataclass(frozen=True)
class LightningMixerConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]


@dataclass(frozen=True)
class GatedFFConfig:
    ff: int


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class PinozenLayerConfig:
    type: str
    mixer: Any
    mlp: Any            # GatedFFConfig or None


def _opt_int(problems, where, obj, key, default, minimum=1):
    if not isinstance(obj, dict) or obj.get(key) is None:
        return default
    return _int(problems, where, obj, key, minimum=minimum)


def _read_rot(problems, where, m) -> PairedRotaryConfig | None:
    rot = m.get("rot") if isinstance(m, dict) else None
    if rot is None:
        return None
    if not isinstance(rot, dict):
        problems.append(f"{where}.rot: expected an object")
        return None
    dims = _int(problems, where + ".rot", rot, "dims", minimum=2)
    if dims % 2:
        problems.append(f"{where}.rot.dims: must be even (got {dims})")
    base = _float(problems, where + ".rot", rot, "base")
    sc = rot.get("scaling")
    scaling = None
    if sc is not None:
        w = where + ".rot.scaling"
        scaling = WavelengthScaling(factor=_float(problems, w, sc, "factor"),
                                    low=_float(problems, w, sc, "low"),
                                    high=_float(problems, w, sc, "high"),
                                    original=_float(problems, w, sc, "original"))
        if scaling.high == scaling.low:
            problems.append(f"{w}: low and high must differ")
    return PairedRotaryConfig(dims, base, scaling)


def _read_left(problems, where, m) -> CappedAttentionConfig:
    if not isinstance(m, dict):
        problems.append(f"{where}: expected an object")
        m = {}
    heads = _int(problems, where, m, "heads")
    kv_heads = _opt_int(problems, where, m, "kv_heads", heads)
    dim = _int(problems, where, m, "dim")
    if heads % kv_heads:
        problems.append(f"{where}: heads={heads} is no multiple of kv_heads={kv_heads}")
    rot = _read_rot(problems, where, m)
    if rot is not None and rot.dims > dim:
        problems.append(f"{where}.rot.dims: {rot.dims} is more than the head's {dim}")
    cap = 0.0
    if m.get("softcap") is not None:
        cap = _float(problems, where, m, "softcap")
    return CappedAttentionConfig(
        heads=heads, kv_heads=kv_heads, dim=dim, vdim=_opt_int(problems, where, m, "vdim", dim),
        scale=_float(problems, where, m, "scale", positive=False),
        conv=_opt_int(problems, where, m, "conv", 0, minimum=0), softcap=cap, rot=rot)


def _read_right(problems, where, m) -> ScanConfig:
    if not isinstance(m, dict):
        problems.append(f"{where}: expected an object")
        m = {}
    return ScanConfig(inner=_int(problems, where, m, "inner"), state=_int(problems, where, m, "state"),
                      dt_rank=_int(problems, where, m, "dt_rank"),
                      conv=_opt_int(problems, where, m, "conv", 0, minimum=0))


def _read_lightning(problems, where, m) -> LightningMixerConfig:
    if not isinstance(m, dict):
        problems.append(f"{where}: expected an object")
        m = {}
    heads = _int(problems, where, m, "heads")
    dim = _int(problems, where, m, "dim")
    decay = m.get("decay")
    ok = isinstance(decay, list) and all(isinstance(x, (int, float)) and not isinstance(x, bool)
                                         for x in decay)
    if not ok or len(decay) != heads:
        problems.append(f"{where}.decay: expected {heads} numbers (one per head), got {decay!r}")
        decay = [1.0] * heads
    return LightningMixerConfig(heads=heads, dim=dim, vdim=_opt_int(problems, where, m, "vdim", dim),
                                decay=tuple(float(x) for x in decay))


def _read_mlp(problems, where, f):
    if f is None:
        return None
    if not isinstance(f, dict) or f.get("kind") not in MLP_KINDS:
        problems.append(f"{where}.kind: unknown feed-forward "
                        f"{f.get('kind') if isinstance(f, dict) else f!r} "
                        f"(known: {list(MLP_KINDS)}, or null)")
        return None
    return GatedFFConfig(ff=_int(problems, where, f, "ff"))


@dataclass(frozen=True)
class PinozenConfig:
    architecture = "pinozen"

    vocab_size: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    max_positions: int | None         # rows of the position table (None: the weight file's shape)
    loop: LoopConfig | None
    layers: tuple[PinozenLayerConfig, ...]
    name: str = "model"

    @classmethod
    def from_json(cls, obj: dict) -> "PinozenConfig":
        if not isinstance(obj, dict):
            raise ConfigError("config.json must hold a JSON object")
        problems: list[str] = []
        vocab = _int(problems, "config", obj, "vocab")
        width = _int(problems, "config", obj, "width")
        eps = _float(problems, "norm", obj.get("norm"), "eps")
        scale = 1.0
        if obj.get("embedding") is not None:
            scale = _float(problems, "embedding", obj.get("embedding"), "scale", positive=False)
        logit_scale = 1.0
        if obj.get("logit_scale") is not None:
            logit_scale = _float(problems, "config", obj, "logit_scale", positive=False)
        max_pos = _opt_int(problems, "config", obj, "max_positions", None)
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
            m = entry.get("mixer")
            if kind == "parallel":
                m = m if isinstance(m, dict) else {}
                mixer = PairMixerConfig(_read_left(problems, where + ".mixer.left", m.get("left")),
                                        _read_right(problems, where + ".mixer.right", m.get("right")))
            else:
                mixer = _read_lightning(problems, where + ".mixer", m)
            layers.append(PinozenLayerConfig(kind, mixer, _read_mlp(problems, where + ".mlp",
                                                                    entry.get("mlp"))))
        loop = None
        if obj.get("loop") is not None:
            lp = obj.get("loop")
            loop = LoopConfig(start=_int(problems, "loop", lp, "start", minimum=0),
                              stop=_int(problems, "loop", lp, "stop", minimum=0),
                              times=_int(problems, "loop", lp, "times", minimum=1))
            if not loop.start < loop.stop <= len(raw_layers):
                problems.append(f"loop: layers {loop.start} .. {loop.stop - 1} are not a stretch "
                                f"of the {len(raw_layers)} layers")
        if problems:
            raise ConfigError("bad config.json: " + "; ".join(problems))
        return cls(vocab_size=vocab, width=width, norm_eps=eps, embedding_scale=scale,
                   logit_scale=logit_scale, max_positions=max_pos, loop=loop, layers=tuple(layers),
                   name=str(obj.get("name", "model")))

    def with_shapes(self, shapes: dict) -> "PinozenConfig":
        """The sizes that only the weight file knows (``{name: shape}``): the rows of the
        position table when config.json does not say."""
        if self.max_positions is None and shapes.get("pos") is not None:
            return replace(self, max_positions=int(shapes["pos"][0]))
        return self

    def run_order(self) -> tuple[tuple[int, bool], ...]:
        """``(layer, first of a pass)`` in the order the layers run: the stretch ``start ..
        stop - 1`` runs ``times`` times in a row with the same weights."""
        n = len(self.layers)
        if self.loop is None:
            return tuple((i, False) for i in range(n))
        lp = self.loop
        order = [(i, False) for i in range(lp.start)]
        for _ in range(lp.times):
            order += [(i, i == lp.start) for i in range(lp.start, lp.stop)]
        return tuple(order + [(i, False) for i in range(lp.stop, n)])

    def n_params(self, *_unused) -> int:
        D = self.width
        total = self.vocab_size * D + D + (self.max_positions or 0) * D
        if self.loop is not None:
            total += 2 * D * D
        for l in self.layers:
            total += D if l.mlp is None else 2 * D + 3 * l.mlp.ff * D
            if l.type == "parallel":
                a, s = l.mixer.left, l.mixer.right
                ch = a.heads * a.dim + a.kv_heads * a.dim + a.kv_heads * a.vdim
                total += ch * D + ch * a.conv + a.heads + a.heads * a.vdim * D + 2 * D
                total += 2 * s.inner * D + s.inner * s.conv + (s.inner if s.conv else 0)
                total += (s.dt_rank + 2 * s.state) * s.inner + s.inner * s.dt_rank
                total += 2 * s.inner + s.inner * s.state + s.inner * D
            else:
                m = l.mixer
                total += 2 * m.heads * m.dim * D + 3 * m.heads * m.vdim * D + m.heads * m.vdim
        return total

    def to_json(self) -> dict[str, Any]:
        out = []
        for l in self.layers:
            if l.type == "parallel":
                a, s = l.mixer.left, l.mixer.right
                left: dict[str, Any] = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim,
                                        "vdim": a.vdim, "scale": a.scale}
                if a.conv:
                    left["conv"] = a.conv
                if a.softcap:
                    left["softcap"] = a.softcap
                if a.rot is not None:
                    left["rot"] = {"dims": a.rot.dims, "base": a.rot.base}
                    if a.rot.scaling is not None:
                        sc = a.rot.scaling
                        left["rot"]["scaling"] = {"factor": sc.factor, "low": sc.low,
                                                  "high": sc.high, "original": sc.original}
                right: dict[str, Any] = {"inner": s.inner, "state": s.state, "dt_rank": s.dt_rank}
                if s.conv:
                    right["conv"] = s.conv
                mx: dict[str, Any] = {"left": left, "right": right}
            else:
                m = l.mixer
                mx = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "decay": list(m.decay)}
            ff = None if l.mlp is None else {"kind": "dense", "ff": l.mlp.ff}
            out.append({"type": l.type, "mixer": mx, "mlp": ff})
        obj: dict[str, Any] = {"architecture": "Pinozen", "name": self.name, "vocab": self.vocab_size,
                               "width": self.width, "norm": {"eps": self.norm_eps},
                               "embedding": {"scale": self.embedding_scale},
                               "logit_scale": self.logit_scale, "layers": out}
        if self.max_positions is not None:
            obj["max_positions"] = self.max_positions
        if self.loop is not None:
            obj["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return obj
