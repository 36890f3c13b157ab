"""Small Lulizen configurations with random weights for the tests, made here (own drawing of the
values; the weight file is written by the Runesun tests' own writer) so that the engine reads
them as it reads any model folder and the plain implementation gets the very same numbers as a
dict."""
from __future__ import annotations

import math
from pathlib import Path

import torch

from runesun_models import write_model


def mixer(heads, kv_heads, dim, scale, vdim=None, softcap=None, rot=None, mask=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim or dim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if mask is not None:
        m["mask"] = mask
    return m


def blocks(size):
    return {"size": size}


def window(size, keep_first=None):
    return {"size": size, **({} if keep_first is None else {"keep_first": keep_first})}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit=None, scale=None, groups=None, shared=None, correction=True):
    router = {"experts": experts, "top": top}
    if scale is not None:
        router["scale"] = scale
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    if not correction:
        router["correction"] = False
    f = {"kind": "moe", "expert": {"ff": ff, **({} if limit is None else {"limit": limit})},
         "router": router}
    if shared is not None:
        f["shared"] = {"ff": shared[0], **({} if shared[1] is None else {"limit": shared[1]})}
    return f


def layer(kind, mx, mlp, weights_of=None):
    out = {"type": kind, "mixer": mx, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


_A1 = layer("attention", mixer(3, 3, 16, 0.25, softcap=30.0, rot=(16, 1000.0), mask=blocks(11)),
            moe(6, 2, 20, limit=1.5, scale=2.5, groups=(3, 2), shared=(24, 0.7)))
# A: odd sizes; values wider than keys (two stores); part of a head rotated; a window shorter
#    than a page that keeps three first tokens; blocks of 11; grouped experts with a shared one;
#    a layer that runs with another's tensors; a layer without feed-forward and without kept
#    tokens
# B: multiples of 16 (the tensor-core paths): heads of 64 with values of 64 over two key heads, a
#    window longer than a page, blocks that straddle pages, groups of two experts (a group's
#    score is all of it), no shared expert, the layers with shared tensors apart from each other
# C: the smallest of everything: one head of two numbers, no cap, no rotation, no mask, no second
#    table, two experts of which one is chosen, a window of one token
# D: nothing a multiple of 8; values narrower than keys; more kept tokens than the window is
#    wide; blocks of one position (a token sees itself and the sink); every expert chosen; no
#    choice bias; no bounds in the experts
CONFIGS = {
    "A": {"architecture": "Lulizen", "vocab": 211, "width": 56, "norm": {"eps": 3e-5},
          "embedding": {"bigram": {"buckets": 97, "mul_prev": 7, "mul_cur": 13}}, "layers": [
        layer("attention_2", mixer(4, 2, 12, 0.3, vdim=20, softcap=8.0, rot=(8, 40.0),
                                   mask=window(9, 3)), dense(40)),
        _A1,
        layer(_A1["type"], _A1["mixer"], _A1["mlp"], weights_of=1),
        layer("attention_2", mixer(2, 1, 24, 0.2, softcap=5.0, rot=(24, 300.0), mask=window(40)), None),
    ]},
    "B": {"architecture": "Lulizen", "vocab": 320, "width": 128, "norm": {"eps": 1e-6},
          "embedding": {"bigram": {"buckets": 128, "mul_prev": 3, "mul_cur": 5}}, "layers": [
        layer("attention_2", mixer(4, 2, 64, 0.125, softcap=20.0, rot=(32, 10000.0),
                                   mask=window(100, 5)), moe(8, 3, 32, limit=2.0, scale=1.0, groups=(4, 2))),
        layer("attention", mixer(4, 4, 32, 0.18, softcap=15.0, rot=(32, 500.0), mask=blocks(70)),
              dense(256)),
        layer("attention_2", mixer(4, 2, 64, 0.125, softcap=20.0, rot=(32, 10000.0),
                                   mask=window(100, 5)), moe(8, 3, 32, limit=2.0, scale=1.0, groups=(4, 2)),
              weights_of=0),
        layer("attention", mixer(2, 1, 128, 0.09, vdim=128, rot=(64, 100000.0), mask=blocks(128)),
              moe(4, 2, 64, limit=1.0, shared=(64, 3.0))),
    ]},
    "C": {"architecture": "Lulizen", "vocab": 29, "width": 8, "norm": {"eps": 1e-5}, "layers": [
        layer("attention", mixer(1, 1, 2, 1.0), moe(2, 1, 3, limit=0.5)),
        layer("attention_2", mixer(2, 1, 4, 0.7, rot=(2, 10.0), mask=window(1, 1)), dense(1)),
        layer("attention_2", mixer(1, 1, 3, 0.5), None),
    ]},
    "D": {"architecture": "Lulizen", "vocab": 99, "width": 44, "norm": {"eps": 1e-6},
          "embedding": {"bigram": {"buckets": 1, "mul_prev": 1, "mul_cur": 1}}, "layers": [
        layer("attention", mixer(6, 2, 10, 0.33, vdim=6, softcap=5.0, rot=(6, 77.0), mask=blocks(1)),
              moe(5, 5, 9, scale=0.5, correction=False)),
        layer("attention_2", mixer(5, 5, 7, 0.4, vdim=9, rot=(4, 20.0), mask=window(3, 10)),
              moe(9, 4, 7, limit=1.0, scale=3.0, groups=(3, 2), shared=(11, None))),
    ]},
}
SEEDS = {"A": 31, "B": 32, "C": 33, "D": 34}


def make_tensors(cfg: dict, seed: int, sink_std: float = 1.5) -> dict[str, torch.Tensor]:
    """fp32 tensors whose values are exact in bfloat16."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * s + mean).to(torch.bfloat16).float()

    def expert(p, hidden):
        out[p + "gate"] = rnd(hidden, D, s=2.0 / math.sqrt(D))
        out[p + "up"] = rnd(hidden, D, s=2.0 / math.sqrt(D))
        out[p + "down"] = rnd(D, hidden, s=1.0 / math.sqrt(hidden))

    D, V = cfg["width"], cfg["vocab"]
    out = {"embed": rnd(V, D)}
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        out["bigram"] = rnd(bg["buckets"] + 1, D, s=0.7)
    for i, l in enumerate(cfg["layers"]):
        if l.get("weights_of") is not None:
            continue
        m, ff, p = l["mixer"], l["mlp"], f"l{i}."
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if ff else ()):
            out[p + n] = rnd(D, s=0.2, mean=1.0)
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
            out[p + "mix." + n] = rnd(rows, D, s=1.5 / math.sqrt(D))
        if l["type"] == "attention":
            out[p + "mix.q.norm"] = rnd(d, s=0.2, mean=1.0)
            out[p + "mix.k.norm"] = rnd(d, s=0.2, mean=1.0)
            out[p + "mix.sink"] = rnd(H, s=sink_std)
        else:
            out[p + "mix.g"] = rnd(H, D, s=2.0 / math.sqrt(D))
        out[p + "mix.o"] = rnd(D, H * dv, s=1 / math.sqrt(H * dv))
        if not ff:
            continue
        if ff["kind"] == "dense":
            expert(p + "mlp.", ff["ff"])
        else:
            r = ff["router"]
            for k in range(r["experts"]):
                expert(f"{p}mlp.e{k}.", ff["expert"]["ff"])
            out[p + "mlp.router"] = rnd(r["experts"], D, s=2.0 / math.sqrt(D))
            if r.get("correction", True):
                out[p + "mlp.correction"] = rnd(r["experts"], s=0.3)
            if ff.get("shared"):
                expert(p + "mlp.shared.", ff["shared"]["ff"])
    out["final.norm"] = rnd(D, s=0.2, mean=1.0)
    out["head"] = rnd(V, D, s=1.0 / math.sqrt(D))
    return out


def make(root: Path, name: str):
    """``(folder, config, tensors)`` of configuration ``name``."""
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, SEEDS[name])
    return write_model(Path(root) / f"lulizen_{name}", cfg, tensors), cfg, tensors
