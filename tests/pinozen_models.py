"""Small Pinozen configurations with random weights for the tests, made here (own drawing of
the values; the weight file is written by the Runesun tests' own writer) so that the engine
reads them as it reads any model folder and the plain implementation gets the very same numbers
as a dict."""
from __future__ import annotations

import math
from pathlib import Path

import torch

from runesun_models import write_model


def left(heads, kv_heads, dim, scale, vdim=None, conv=None, softcap=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim or dim, "scale": scale}
    if conv is not None:
        m["conv"] = conv
    if softcap is not None:
        m["softcap"] = softcap
    if rot is not None:
        m["rot"] = rot
    return m


def right(inner, state, dt_rank, conv=None):
    m = {"inner": inner, "state": state, "dt_rank": dt_rank}
    if conv is not None:
        m["conv"] = conv
    return m


def pair(l, r, mlp=None):
    return {"type": "parallel", "mixer": {"left": l, "right": r}, "mlp": mlp}


def lightning(heads, dim, decay, vdim=None, mlp=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim or dim,
                                           "decay": list(decay)}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


# A: odd sizes; values wider than keys; part of a head rotated with scaled frequencies that hit
#    all three ranges of wavelength; convolutions of 3 and 5 taps; a stretch of two layers that
#    runs twice, starting with the lightning layer; a layer without feed-forward
# B: multiples of 16 (the tensor-core paths), keys of 64 with equal values, a whole head
#    rotated without scaling, no cap on the scores, a stretch of one layer three times
# C: the smallest of everything: one head of two numbers, a state of one, a convolution of one
#    tap and one without, no loop, no scales, no rotation
# D: nothing a multiple of 8; values narrower than keys; a convolution of two taps; the loop
#    is the whole model; a rank and a state that are no powers of two
CONFIGS = {
    "A": {"architecture": "Pinozen", "vocab": 211, "width": 56, "max_positions": 320,
          "norm": {"eps": 3e-5}, "embedding": {"scale": 5.0}, "logit_scale": 0.5,
          "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [
        pair(left(4, 2, 12, 0.3, vdim=20, conv=3, softcap=8.0, rot=rot(8, 40.0, (6.0, 1.0, 3.0, 48))),
             right(40, 5, 3, conv=5), mlp=dense(72)),
        lightning(3, 10, (0.5, 0.9, 0.99), vdim=14, mlp=None),
        pair(left(3, 3, 16, 0.25, conv=4, softcap=30.0, rot=rot(16, 1000.0)),
             right(24, 9, 4, conv=3), mlp=dense(40)),
        lightning(2, 24, (0.8, 1.0), mlp=dense(32)),
    ]},
    "B": {"architecture": "Pinozen", "vocab": 320, "width": 128, "max_positions": 512,
          "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "logit_scale": 1.0,
          "loop": {"start": 0, "stop": 1, "times": 3}, "layers": [
        pair(left(4, 1, 64, 0.125, conv=4, rot=rot(64, 10000.0)), right(256, 16, 8, conv=4),
             mlp=dense(256)),
        lightning(4, 32, (0.7, 0.9, 0.97, 0.995), vdim=64, mlp=dense(128)),
        pair(left(8, 4, 32, 0.18, softcap=15.0, conv=2, rot=rot(16, 500.0, (4.0, 1.0, 4.0, 64))),
             right(128, 32, 16, conv=2), mlp=None),
    ]},
    "C": {"architecture": "Pinozen", "vocab": 29, "width": 8, "max_positions": 200,
          "norm": {"eps": 1e-5}, "layers": [
        pair(left(1, 1, 2, 1.0, conv=1), right(4, 1, 1), mlp=dense(1)),
        lightning(1, 1, (0.9,), mlp=None),
        pair(left(2, 1, 3, 0.7, softcap=2.0), right(2, 2, 1, conv=2), mlp=dense(5)),
    ]},
    "D": {"architecture": "Pinozen", "vocab": 99, "width": 44, "max_positions": 256,
          "norm": {"eps": 1e-6}, "embedding": {"scale": 7.0}, "logit_scale": 2.0,
          "loop": {"start": 0, "stop": 2, "times": 2}, "layers": [
        lightning(5, 7, (0.3, 0.6, 0.9, 0.95, 0.999), vdim=9, mlp=dense(30)),
        pair(left(6, 2, 10, 0.33, vdim=6, conv=2, softcap=5.0, rot=rot(6, 77.0, (2.0, 2.0, 5.0, 20))),
             right(50, 11, 7, conv=6), mlp=dense(20)),
    ]},
}
SEEDS = {"A": 21, "B": 22, "C": 23, "D": 24}


def make_tensors(cfg: dict, seed: int, sink_std: float = 1.5) -> dict[str, torch.Tensor]:
    """fp32 tensors whose values are exact in bfloat16."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * s + mean).to(torch.bfloat16).float()

    D, V = cfg["width"], cfg["vocab"]
    scale = (cfg.get("embedding") or {}).get("scale", 1.0)
    out = {"embed": rnd(V, D, s=1.0 / scale), "pos": rnd(cfg["max_positions"], D, s=0.4)}
    if cfg.get("loop"):
        out["loop.in"] = (torch.cat([torch.eye(D), torch.zeros(D, D)], 1)
                          + torch.randn(D, 2 * D, generator=g) * (0.5 / math.sqrt(2 * D))
                          ).to(torch.bfloat16).float()
    for i, l in enumerate(cfg["layers"]):
        m, ff, p = l["mixer"], l["mlp"], f"l{i}."
        out[p + "norm1"] = rnd(D, s=0.2, mean=1.0)
        if l["type"] == "parallel":
            a, s = m["left"], m["right"]
            H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            lp, rp = p + "mix.left.", p + "mix.right."
            for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                out[lp + n] = rnd(rows, D, s=1.5 / math.sqrt(D))
                if a.get("conv"):
                    out[lp + n + ".conv"] = rnd(rows, a["conv"], s=0.7)
            out[lp + "sink"] = rnd(H, s=sink_std)
            out[lp + "o"] = rnd(D, H * dv, s=1 / math.sqrt(H * dv))
            out[lp + "out"] = rnd(D, s=0.2, mean=1.0)
            I, N, R = s["inner"], s["state"], s["dt_rank"]
            out[rp + "in"] = rnd(2 * I, D, s=1.5 / math.sqrt(D))
            if s.get("conv"):
                out[rp + "conv"] = rnd(I, s["conv"], s=0.7)
                out[rp + "conv.b"] = rnd(I, s=0.3)
            out[rp + "x"] = rnd(R + 2 * N, I, s=1.5 / math.sqrt(I))
            out[rp + "dt"] = rnd(I, R, s=1.0 / math.sqrt(R))
            out[rp + "dt.b"] = rnd(I, s=1.0, mean=-2.0)
            out[rp + "A_log"] = rnd(I, N, s=0.7, mean=-0.5)
            out[rp + "D"] = rnd(I, s=0.3, mean=1.0)
            out[rp + "o"] = rnd(D, I, s=1 / math.sqrt(I))
            out[rp + "out"] = rnd(D, s=0.2, mean=1.0)
        else:
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            out[p + "mix.q"] = rnd(H * d, D, s=1.5 / math.sqrt(D))
            out[p + "mix.k"] = rnd(H * d, D, s=1.5 / math.sqrt(D))
            out[p + "mix.v"] = rnd(H * dv, D, s=1.5 / math.sqrt(D))
            out[p + "mix.g"] = rnd(H * dv, D, s=1.5 / math.sqrt(D))
            out[p + "mix.o"] = rnd(D, H * dv, s=1 / math.sqrt(H * dv))
            out[p + "mix.norm"] = rnd(H * dv, s=0.2, mean=1.0)
        if ff:
            out[p + "norm2"] = rnd(D, s=0.2, mean=1.0)
            out[p + "mlp.gate"] = rnd(ff["ff"], D, s=1.5 / math.sqrt(D))
            out[p + "mlp.up"] = rnd(ff["ff"], D, s=1.5 / math.sqrt(D))
            out[p + "mlp.down"] = rnd(D, ff["ff"], s=1 / math.sqrt(ff["ff"]))
    out["final.norm"] = rnd(D, s=0.2, mean=1.0)
    return out


def make(root: Path, name: str):
    """``(folder, config, tensors)`` of configuration ``name``."""
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, SEEDS[name])
    return write_model(Path(root) / f"pinozen_{name}", cfg, tensors), cfg, tensors
