"""Pinozen as data: how its configuration maps onto parts, and where its parameters are found
in a weight file.  This is the only file that knows the architecture.

Structure: token embedding times a constant plus a learned position row; pre-norm layers (RMS
norms) of two kinds in any order, ``parallel`` (an attention branch with short convolutions,
paired rotation, capped scores and a sink beside a selective-scan branch, their normed results
averaged) and ``lightning`` (linear attention with a fixed decay per head); a gated dense
feed-forward with relu, or none; a stretch of layers that runs several times in a row with the
same weights, each pass with storage of its own and entered through one matrix on the stream
beside the embedding's output; a final RMS norm, the embedding table as the output head, and a
constant on the logits.

Tensor names: ``embed``, ``pos``, ``loop.in``, ``final.norm``, and per layer ``l<i>.``:
``norm1``, ``norm2``, ``mix.left.{q, k, v, q.conv, k.conv, v.conv, sink, o, out}`` with
``mix.right.{in, conv, conv.b, x, dt, dt.b, A_log, D, o, out}``, or ``mix.{q, k, v, g, o,
norm}``, and ``mlp.{gate, up, down}``; every linear weight stored ``(out, in)``.
"""
from __future__ import annotations

import math

import torch

from ..config.pinozen import PinozenConfig
from ..config.registry import Architecture, register_architecture
from ..engine.spec import LayerSpec, ModelSpec
from ..parts.base import PartSpec
from ..weights.loader import Recipe, Source, WeightPlan, take
from .runesun import _rows

DEFAULT_MAX_POSITIONS = 2048     # of a model made here without a weight file to give it


def _max_positions(cfg: PinozenConfig) -> int:
    return cfg.max_positions if cfg.max_positions is not None else DEFAULT_MAX_POSITIONS


def build_spec(cfg: PinozenConfig) -> ModelSpec:
    D = cfg.width
    norm = PartSpec("rmsnorm", {"width": D, "eps": cfg.norm_eps})
    layers = []
    for l in cfg.layers:
        mx, ff = l.mixer, l.mlp
        if l.type == "parallel":
            a, s = mx.left, mx.right
            rot = a.rot
            scaling = None if rot is None or rot.scaling is None else {
                "factor": rot.scaling.factor, "low": rot.scaling.low, "high": rot.scaling.high,
                "original": rot.scaling.original}
            left = PartSpec("capped_attention", {
                "width": D, "n_heads": a.heads, "n_kv_heads": a.kv_heads, "head_dim": a.dim,
                "value_dim": a.vdim, "scale": a.scale, "conv": a.conv, "softcap": a.softcap,
                "sink": True, "rot_dims": 0 if rot is None else rot.dims,
                "rot_base": 10000.0 if rot is None else rot.base, "rot_scaling": scaling})
            right = PartSpec("selective_scan", {
                "width": D, "inner": s.inner, "n_state": s.state, "dt_rank": s.dt_rank,
                "conv": s.conv})
            mixer = PartSpec("normed_pair", {"width": D, "eps": cfg.norm_eps, "left": left,
                                             "right": right, "coef": 0.5})
        else:
            mixer = PartSpec("decayed_linear_attention", {
                "width": D, "n_heads": mx.heads, "head_dim": mx.dim, "value_dim": mx.vdim,
                "decay": tuple(mx.decay), "eps": cfg.norm_eps})
        ffn = None if ff is None else PartSpec("gated_mlp", {"width": D, "hidden": ff.ff,
                                                             "activation": "relu"})
        layers.append(LayerSpec(mixer=mixer, ffn=ffn, norm_mixer=norm,
                                norm_ffn=None if ffn is None else norm, block=PartSpec("pre_norm")))
    order = cfg.run_order()
    return ModelSpec(
        architecture="pinozen", vocab_size=cfg.vocab_size, width=D,
        max_seq_len=_max_positions(cfg),
        position=PartSpec("learned_absolute", {"max_positions": _max_positions(cfg), "width": D}),
        layers=tuple(layers), final_norm=norm, tie_head=True,
        schedule=tuple(i for i, _ in order), embedding_scale=cfg.embedding_scale,
        logit_scale=cfg.logit_scale,
        stream_input=None if cfg.loop is None else PartSpec("embedding_remix", {"width": D}),
        stream_input_before=tuple(e for e, (_, first) in enumerate(order) if first))


def _halves(names_shapes, half: int) -> Recipe:
    """Two ``(n, in)`` matrices one under the other, each followed by rows of zeros up to
    ``half`` rows (a gated feed-forward's two first products side by side)."""
    srcs = [Source(n, (tuple(s),)) for n, s in names_shapes]

    def combine(ts):
        if len({t.dtype for t in ts}) > 1:
            ts = [t.to(torch.float32) for t in ts]
        parts = []
        for t in ts:
            parts.append(t)
            if half > t.shape[0]:
                parts.append(torch.zeros((half - t.shape[0], t.shape[1]), dtype=t.dtype))
        return torch.cat(parts, dim=0).contiguous()

    return Recipe(srcs, combine)


def weight_plan(cfg: PinozenConfig, spec: ModelSpec, names: set[str]) -> WeightPlan:
    D, V = cfg.width, cfg.vocab_size
    r: dict[str, Recipe] = {"embedding.table": take("embed", (V, D)),
                            "position.table": take("pos", (_max_positions(cfg), D)),
                            "final_norm.weight": take("final.norm", (D,))}
    if cfg.loop is not None:
        r["stream_input.proj.weight"] = take("loop.in", (D, 2 * D))
    for i, l in enumerate(cfg.layers):
        mx, ff = l.mixer, l.mlp
        p, L = f"l{i}.", f"layers.{i}."
        r[L + "norm_mixer.weight"] = take(p + "norm1", (D,))
        if l.type == "parallel":
            a, s = mx.left, mx.right
            q, k, v = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
            lp, rp = p + "mix.left.", p + "mix.right."
            r[L + "mixer.left.proj.weight"] = _rows(
                [(lp + "q", (q, D)), (lp + "k", (k, D)), (lp + "v", (v, D))], multiple=8)
            if a.conv:
                r[L + "mixer.left.conv"] = _rows(
                    [(lp + "q.conv", (q, a.conv)), (lp + "k.conv", (k, a.conv)),
                     (lp + "v.conv", (v, a.conv))])
            r[L + "mixer.left.sink"] = take(lp + "sink", (a.heads,))
            r[L + "mixer.left.out.weight"] = take(lp + "o", (D, a.heads * a.vdim))
            r[L + "mixer.left_norm"] = take(lp + "out", (D,))
            r[L + "mixer.right.in_proj.weight"] = take(rp + "in", (2 * s.inner, D))
            if s.conv:
                r[L + "mixer.right.conv"] = take(rp + "conv", (s.inner, s.conv))
                r[L + "mixer.right.conv_bias"] = take(rp + "conv.b", (s.inner,))
            r[L + "mixer.right.x_proj.weight"] = _rows(
                [(rp + "x", (s.dt_rank + 2 * s.state, s.inner))], multiple=8)
            r[L + "mixer.right.dt_proj.weight"] = take(rp + "dt", (s.inner, s.dt_rank))
            r[L + "mixer.right.dt_bias"] = take(rp + "dt.b", (s.inner,))
            r[L + "mixer.right.a_log"] = take(rp + "A_log", (s.inner, s.state))
            r[L + "mixer.right.d_skip"] = take(rp + "D", (s.inner,))
            r[L + "mixer.right.out.weight"] = take(rp + "o", (D, s.inner))
            r[L + "mixer.right_norm"] = take(rp + "out", (D,))
        else:
            qk, vw = mx.heads * mx.dim, mx.heads * mx.vdim
            r[L + "mixer.proj.weight"] = _rows(
                [(p + "mix.q", (qk, D)), (p + "mix.k", (qk, D)), (p + "mix.v", (vw, D)),
                 (p + "mix.g", (vw, D))], multiple=8)
            r[L + "mixer.norm"] = take(p + "mix.norm", (vw,))
            r[L + "mixer.out.weight"] = take(p + "mix.o", (D, vw))
        if ff is not None:
            half = -(-ff.ff // 8) * 8
            r[L + "norm_ffn.weight"] = take(p + "norm2", (D,))
            r[L + "ffn.fc.weight"] = _halves([(p + "mlp.gate", (ff.ff, D)), (p + "mlp.up", (ff.ff, D))],
                                             half)
            r[L + "ffn.proj.weight"] = take(p + "mlp.down", (D, ff.ff))
    # a layer without a feed-forward may still carry the norm in front of it in the file
    ignored = {f"l{i}.norm2" for i, l in enumerate(cfg.layers) if l.mlp is None}
    return WeightPlan(r, ignored)


def complete_config(cfg: PinozenConfig, shapes: dict) -> PinozenConfig:
    return cfg.with_shapes(shapes)


def random_tensors(cfg: PinozenConfig, seed: int, *, gain: float = 1.0, std: float | None = None,
                   sink_std: float = 1.0, gamma_jitter: float = 0.1, pos_std: float = 0.3,
                   dtype: torch.dtype = torch.bfloat16) -> dict:
    """Random Pinozen tensors under the names of a weight file.  Matrices ~N(0, gain^2 / in) (or
    ~N(0, std^2) if ``std`` is given), embeddings ~N(0, 1) divided by the embedding's scale,
    position rows ~N(0, pos_std^2), norm weights 1 + N(0, gamma_jitter^2), sinks ~N(0,
    sink_std^2), the scan's ``A_log`` the logarithms of 1 .. N with a little noise and its step
    biases such that the step sizes start between 0.001 and 0.1; drawn in fp32 from a seeded CPU
    generator in a fixed order and stored in ``dtype``."""
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))

    def mat(n_out, n_in, s=None):
        s = (gain / math.sqrt(n_in) if std is None else std) if s is None else s
        return (torch.randn(n_out, n_in, generator=g, dtype=torch.float32) * s).to(dtype)

    def vec(n, s, mean=0.0):
        return (torch.randn(n, generator=g, dtype=torch.float32) * s + mean).to(dtype)

    D, V = cfg.width, cfg.vocab_size
    out: dict[str, torch.Tensor] = {
        "embed": mat(V, D, 1.0 / max(abs(cfg.embedding_scale), 1e-6)),
        "pos": mat(_max_positions(cfg), D, pos_std)}
    if cfg.loop is not None:
        # near [I | 0]: a pass starts near where the last one ended
        w = torch.cat([torch.eye(D), torch.zeros(D, D)], dim=1)
        out["loop.in"] = (w + torch.randn(D, 2 * D, generator=g) * (0.3 / math.sqrt(2 * D))).to(dtype)
    for i, l in enumerate(cfg.layers):
        mx, ff = l.mixer, l.mlp
        p = f"l{i}."
        out[p + "norm1"] = vec(D, gamma_jitter, 1.0)
        if l.type == "parallel":
            a, s = mx.left, mx.right
            lp, rp = p + "mix.left.", p + "mix.right."
            for n, rows in (("q", a.heads * a.dim), ("k", a.kv_heads * a.dim), ("v", a.kv_heads * a.vdim)):
                out[lp + n] = mat(rows, D)
                if a.conv:
                    out[lp + n + ".conv"] = mat(rows, a.conv, 1.0 / math.sqrt(a.conv))
            out[lp + "sink"] = vec(a.heads, sink_std)
            out[lp + "o"] = mat(D, a.heads * a.vdim)
            out[lp + "out"] = vec(D, gamma_jitter, 1.0)
            out[rp + "in"] = mat(2 * s.inner, D)
            if s.conv:
                out[rp + "conv"] = mat(s.inner, s.conv, 1.0 / math.sqrt(s.conv))
                out[rp + "conv.b"] = vec(s.inner, 0.1)
            out[rp + "x"] = mat(s.dt_rank + 2 * s.state, s.inner)
            out[rp + "dt"] = mat(s.inner, s.dt_rank)
            step = torch.exp(torch.rand(s.inner, generator=g) * (math.log(0.1) - math.log(0.001))
                             + math.log(0.001))
            out[rp + "dt.b"] = (step + torch.log(-torch.expm1(-step))).to(dtype)   # softplus^-1
            a_log = torch.log(torch.arange(1, s.state + 1, dtype=torch.float32)).repeat(s.inner, 1)
            out[rp + "A_log"] = (a_log + torch.randn(s.inner, s.state, generator=g) * 0.1).to(dtype)
            out[rp + "D"] = vec(s.inner, 0.1, 1.0)
            out[rp + "o"] = mat(D, s.inner)
            out[rp + "out"] = vec(D, gamma_jitter, 1.0)
        else:
            qk, vw = mx.heads * mx.dim, mx.heads * mx.vdim
            out[p + "mix.q"] = mat(qk, D)
            out[p + "mix.k"] = mat(qk, D)
            out[p + "mix.v"] = mat(vw, D)
            out[p + "mix.g"] = mat(vw, D)
            out[p + "mix.o"] = mat(D, vw)
            out[p + "mix.norm"] = vec(vw, gamma_jitter, 1.0)
        if ff is not None:
            out[p + "norm2"] = vec(D, gamma_jitter, 1.0)
            out[p + "mlp.gate"] = mat(ff.ff, D)
            out[p + "mlp.up"] = mat(ff.ff, D)
            out[p + "mlp.down"] = mat(D, ff.ff)
    out["final.norm"] = vec(D, gamma_jitter, 1.0)
    return out


ARCHITECTURE = register_architecture(Architecture(
    name="pinozen", config_cls=PinozenConfig, build_spec=build_spec, weight_plan=weight_plan,
    aliases=("Pinozen",), random_tensors=random_tensors, complete_config=complete_config),
    replace=True)
