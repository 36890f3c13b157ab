"""Lulizen configurations drawn at random (sizes, head counts, layer order, masks, routers, shared
tensors, with and without the second table) through the engine on the GPU against the plain
implementation: three unequal requests in one batch, prompts with every logit wanted, then
decoded together while the shorter ones end, in both precisions."""
import random

import pytest
import torch

import lulizen_models as LM
import plain_lulizen as PL
from test_gpu_lulizen import MARGIN, Routed
from nimbus_infer_rs_b200 import Engine

pytestmark = pytest.mark.gpu
TOL = {"float32": 2e-4, "bfloat16": 8e-2}


def random_config(rng):
    width = rng.choice([64, 100, 128, 192, 96, 328])
    vocab = rng.choice([97, 300, 1000, 450])

    def mixer(kind):
        d = rng.choice([16, 32, 48, 64, 96, 128, 24])
        dv = d if rng.random() < 0.7 else rng.choice([16, 32, 64, 128, 40])
        kv_heads = rng.choice([1, 2, 3, 4])
        m = {"heads": kv_heads * rng.choice([1, 2, 3, 4]), "kv_heads": kv_heads, "dim": d, "vdim": dv,
             "scale": rng.choice([d ** -0.5, 0.1, 0.2])}
        if rng.random() < 0.8:
            m["softcap"] = rng.choice([5.0, 30.0, 40.0])
        if rng.random() < 0.85:
            half = d // 2 if (d // 2) % 2 == 0 else d
            m["rot"] = {"dims": rng.choice([d, half, max(2, (d // 4) // 2 * 2)]),
                        "base": rng.choice([100.0, 10000.0, 1e6])}
        if rng.random() < 0.9:
            m["mask"] = {"size": rng.choice([1, 7, 33, 64, 65, 90, 100, 128, 130, 200, 256])}
            if kind == "attention_2" and rng.random() < 0.8:
                m["mask"]["keep_first"] = rng.choice([0, 1, 3, 5, 64, 65, 70])
        return m

    def mlp():
        r = rng.random()
        if r < 0.15:
            return None
        if r < 0.4:
            return {"kind": "dense", "ff": rng.choice([40, 64, 256, 100])}
        groups, per = rng.choice([1, 2, 3, 4]), rng.choice([1, 2, 3, 4])
        keep = rng.randint(1, groups)
        f = {"kind": "moe", "expert": {"ff": rng.choice([16, 64, 40]), "limit": rng.choice([0.5, 1.0, 7.0])},
             "router": {"experts": groups * per, "top": rng.randint(1, keep * per),
                        "scale": rng.choice([1.0, 1.5, 2.5])}}
        if rng.random() < 0.8:
            f["router"]["groups"] = {"count": groups, "keep": keep}
        elif f["router"]["top"] > f["router"]["experts"]:
            f["router"]["top"] = f["router"]["experts"]
        if rng.random() < 0.7:
            f["shared"] = {"ff": rng.choice([32, 128, 24]), "limit": rng.choice([1.0, 2.0])}
        return f

    layers = []
    for _ in range(rng.randint(2, 6)):
        if layers and rng.random() < 0.25:            # a layer on an earlier layer's tensors
            j = rng.randrange(len(layers))
            while layers[j].get("weights_of") is not None:
                j = layers[j]["weights_of"]
            layers.append({"type": layers[j]["type"], "mixer": layers[j]["mixer"],
                           "mlp": layers[j]["mlp"], "weights_of": j})
        else:
            kind = rng.choice(["attention", "attention_2"])
            layers.append({"type": kind, "mixer": mixer(kind), "mlp": mlp()})
    cfg = {"architecture": "Lulizen", "vocab": vocab, "width": width,
           "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}
    if rng.random() < 0.8:
        cfg["embedding"] = {"bigram": {"buckets": rng.choice([13, 511, 128]),
                                       "mul_prev": rng.choice([29, 3]), "mul_cur": rng.choice([19, 5])}}
    return cfg


def _worst_rows(got, ref):
    got, ref = got.double().cpu(), ref.double().cpu()
    return (got - ref).abs().reshape(got.shape[0], -1).max(1).values / float(ref.abs().max())


@pytest.mark.parametrize("seed", range(12))
def test_a_random_configuration(tmp_path, seed):
    rng = random.Random(seed)
    cfg = random_config(rng)
    P = LM.make_tensors(cfg, seed)
    folder = LM.write_model(tmp_path / "m", cfg, P)
    lens = [rng.choice([300, 140, 70]), rng.choice([1, 9, 66]), rng.choice([130, 200])]
    heads = [max(1, n - rng.choice([3, 20, 40])) for n in lens]
    g = torch.Generator().manual_seed(seed)
    seqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lens]
    for dtype in ("float32", "bfloat16"):
        e = Engine.load(folder, dtype=dtype, cache_tokens=1024)
        e.step_graphs = None
        e.routed = Routed(e)
        slots = [e.alloc_slot() for _ in lens]
        got = {i: [] for i in range(3)}
        out = e.step([(slots[i], seqs[i][:heads[i]], list(range(heads[i]))) for i in range(3)])
        at = 0
        for i in range(3):
            got[i].append(out[at:at + heads[i]])
            at += heads[i]
        k = 0
        while True:
            live = [i for i in range(3) if heads[i] + k < lens[i]]
            if not live:
                break
            out = e.step([(slots[i], [seqs[i][heads[i] + k]], [0]) for i in live])
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
            k += 1
        e.check_errors()
        for i in range(3):
            ref = PL.logits(seqs[i], P, cfg, routed=e.routed.by_slot.get(slots[i]), margin=MARGIN[dtype])
            rows = _worst_rows(torch.cat(got[i]), ref)
            over = int((rows > TOL[dtype]).sum())
            allowed = 0 if dtype == "float32" else max(1, len(rows) // 50)
            assert over <= allowed and float(rows.max()) <= 8 * TOL[dtype], \
                f"{dtype} request {i}: {over} rows over, worst {float(rows.max()):.3e}; {cfg}"
