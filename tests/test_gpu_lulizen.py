"""Lulizen on the GPU against the plain implementation, in 32-bit and in bfloat16: whole prompts,
token by token, portions, unequal batches, slots, pages and state rows used again, long
decoding across windows and blocks, greedy generation through the engine's own loop, and a test
that changes mechanisms in the plain implementation and sees the comparison fail."""
import copy

import pytest
import torch

import lulizen_models as LM
import plain_lulizen as PL
from gpu_helpers import DTYPES
from nimbus_infer_rs_b200 import Engine, SamplingParams

pytestmark = pytest.mark.gpu
NAMES = ["A", "B", "C", "D"]
# Largest |engine - plain| relative to the largest |plain logit| for whole models of this
# design.  Every sublayer's result is normed to unit size before it is added, so a rounding
# error in a small result enters the stream at full size; the mechanisms alone are held to 2e-5
# and 2e-2 in test_gpu_lulizen_kernels.py.
TOL = {"float32": 1e-4, "bfloat16": 5e-2}


def assert_close(got, ref, dtype, what=""):
    """In 32-bit every row within the tolerance.  In bfloat16 one row in fifty (at least one) may
    be over it, none over eight times it."""
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    rows = (got - ref).abs().reshape(got.shape[0], -1).max(dim=1).values / float(ref.abs().max())
    over = int((rows > TOL[dtype]).sum())
    allowed = 0 if dtype == "float32" else max(1, got.shape[0] // 50)
    assert over <= allowed and float(rows.max()) <= 8 * TOL[dtype], \
        f"{what}: {over} rows over {TOL[dtype]:.0e} (allowed {allowed}), worst {float(rows.max()):.3e} " \
        f"at row {int(rows.argmax())}"


def _cases(names):
    """Every configuration in both precisions, except C in bfloat16: its norms over one or two
    numbers are sign functions, which rounding flips."""
    return [(n, d) for n in names for d in DTYPES if not (n == "C" and d == "bfloat16")]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("lulizen")
    return {n: LM.make(root, n) for n in LM.CONFIGS}


def _tokens(vocab, n, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


# A router's choice between experts (or groups of experts) whose scores are closer than this is a
# close call that rounding may settle either way; the plain implementation then follows the
# engine (and insists on its own choice everywhere else).
MARGIN = {"float32": 1e-4, "bfloat16": 0.05}


class Routed:
    """Notes what the router kernel chose, per slot, at every position of every layer run with
    routed experts, for the steps that go through ``Engine.step``."""

    def __init__(self, engine):
        self.by_slot, self._calls = {}, []
        ops, orig, step, alloc = engine.ops, engine.ops.moe_route_sigmoid, engine.step, engine.alloc_slot

        def tapped(logits, col, bias, n_experts, top, *rest):
            orig(logits, col, bias, n_experts, top, *rest)
            self._calls.append(rest[-2].clone())            # idx

        def stepped(entries):
            ops.moe_route_sigmoid = tapped
            try:
                out = step(entries)
            finally:
                del ops.moe_route_sigmoid                    # the class's method is back
            calls, self._calls = [c.cpu().long() for c in self._calls], []
            at = 0
            for e in entries:
                n = len(e[1])
                mine = [c[at:at + n] for c in calls]
                old = self.by_slot.get(e[0])
                self.by_slot[e[0]] = mine if old is None else [torch.cat([a, b]) for a, b in zip(old, mine)]
                at += n
            return out

        def allocated():
            slot = alloc()
            self.by_slot.pop(slot, None)
            return slot

        engine.step, engine.alloc_slot = stepped, allocated


def _engine(models, name, dtype, cache_tokens=1024, tap=True, **kw):
    e = Engine.load(models[name][0], dtype=dtype, cache_tokens=cache_tokens, **kw)
    if tap:
        e.step_graphs = None               # every launch goes through Python: the tap sees it
        e.routed = Routed(e)
    return e


def _plain(e, slot, toks, P, cfg, dtype):
    """The plain logits of the sequence in ``slot``, close calls of the routers settled as the
    engine settled them."""
    return PL.logits(toks, P, cfg, routed=e.routed.by_slot.get(slot), margin=MARGIN[dtype])


@pytest.mark.parametrize("name,dtype", _cases(NAMES))
def test_each_request_alone_and_whole(models, name, dtype):
    _, cfg, P = models[name]
    e = _engine(models, name, dtype)
    for i, n in enumerate((1, 2, 33, 64, 65, 190)):
        toks = _tokens(cfg["vocab"], n, 10 + i)
        s = e.alloc_slot()
        out = e.step([(s, toks, list(range(n)))])
        assert_close(out, _plain(e, s, toks, P, cfg, dtype), dtype, f"{name} whole, {n} tokens")
        e.free_slot(s)
    e.check_errors()


def test_layer_by_layer_in_32_bit(models):
    _, cfg, P = models["A"]
    e = _engine(models, "A", "float32")
    e.step_graphs = None
    assert e.model.run_order == (0, 1, 1, 2)
    snaps = []
    for layer in e.model.layers:
        f = layer.block.forward
        layer.block.forward = lambda ctx, x, l, f=f: (f(ctx, x, l), snaps.append(x.clone()))[0]
    toks = _tokens(211, 90, 5)
    e.step([(e.alloc_slot(), toks, [0])])
    ref = PL.hidden_states(toks, P, cfg)
    assert len(snaps) == ref.shape[0]
    for i, (got, want) in enumerate(zip(snaps, ref)):
        assert_close(got[:90], want, "float32", f"stream after layer run {i}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_recorded_steps_give_what_plain_launches_give(models, name, dtype):
    """A step whose shape comes again is replayed from a CUDA graph: bit for bit the same."""
    _, cfg, _ = models[name]
    e, plainly = _engine(models, name, dtype, tap=False), _engine(models, name, dtype, tap=False)
    plainly.step_graphs = None
    for n in (1, 70, 1, 70, 1, 70):
        toks = _tokens(cfg["vocab"], n, n)
        s, t = e.alloc_slot(), plainly.alloc_slot()
        a, b = e.step([(s, toks, list(range(n)))]), plainly.step([(t, toks, list(range(n)))])
        for k in range(3):
            a = torch.cat([a, e.step([(s, [k + 1], [0])])])
            b = torch.cat([b, plainly.step([(t, [k + 1], [0])])])
        e.free_slot(s)
        plainly.free_slot(t)
        assert torch.equal(a, b)
    assert e.step_graphs.replays > 0


@pytest.mark.parametrize("name,dtype", _cases(NAMES))
def test_last_tokens_one_by_one(models, name, dtype):
    """Prefill, then decoding through the caches and the state rows."""
    _, cfg, P = models[name]
    e = _engine(models, name, dtype)
    for n, head in ((34, 1), (190, 140)):
        toks = _tokens(cfg["vocab"], n, n)
        s = e.alloc_slot()
        outs = [e.step([(s, toks[:head], [head - 1])])]
        for t in range(head, n):
            outs.append(e.step([(s, [toks[t]], [0])]))
        e.free_slot(s)
        assert_close(torch.cat(outs), _plain(e, s, toks, P, cfg, dtype)[head - 1:], dtype, f"{name} from {head} of {n}")


@pytest.mark.parametrize("name,dtype", _cases(["A", "B", "D"]))
def test_portions_of_several_sizes(models, name, dtype):
    """Portions that start inside a window, inside a block and right after the kept tokens, ending
    on and beside page ends."""
    _, cfg, P = models[name]
    e = _engine(models, name, dtype)
    toks = _tokens(cfg["vocab"], 203, 3)
    s, at, outs = e.alloc_slot(), 0, []
    for size in (2, 61, 1, 2, 64, 3, 70):
        outs.append(e.step([(s, toks[at:at + size], list(range(size)))]))
        at += size
    assert_close(torch.cat(outs), _plain(e, s, toks, P, cfg, dtype), dtype, f"{name} portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_batches_on_slots_and_pages_used_again(models, name, dtype):
    """Batches of unequal prompts, decoded together while the shorter ones end; the cache holds
    one batch, so the next one gets the same slots, pages and state rows."""
    _, cfg, P = models[name]
    e = _engine(models, name, dtype, cache_tokens=6 * 64, n_slots=3)
    V = cfg["vocab"]
    for turn, lens in enumerate(((130, 7, 66), (64, 129, 2), (1, 1, 190))):
        seqs = [_tokens(V, n, 31 * turn + i) for i, n in enumerate(lens)]
        heads = [max(1, n - 3 - 2 * i) for i, n in enumerate(lens)]
        slots = [e.alloc_slot() for _ in lens]
        got = {i: [] for i in range(3)}
        out = e.step([(slots[i], t[:h], [0, h - 1]) for i, (t, h) in enumerate(zip(seqs, heads))])
        for i in range(3):
            got[i] += [out[2 * i], out[2 * i + 1]]
        k = 0
        while True:
            live = [i for i in range(3) if heads[i] + k < lens[i]]
            if not live:
                break
            out = e.step([(slots[i], [seqs[i][heads[i] + k]], [0]) for i in live])
            for j, i in enumerate(live):
                got[i].append(out[j])
            k += 1
        for i in range(3):
            ref = _plain(e, slots[i], seqs[i], P, cfg, dtype)
            places = [0, heads[i] - 1] + list(range(heads[i], lens[i]))
            assert_close(torch.stack(got[i]), ref[places], dtype, f"{name} batch {turn} request {i}")
            e.free_slot(slots[i])
    assert all(g.pool.n_free == g.pool.n_pages for g in e.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "D"])
def test_long_decoding_from_the_first_token(models, name, dtype):
    """Windows and blocks pass over decoded tokens; pages behind them are given back."""
    _, cfg, P = models[name]
    e = _engine(models, name, dtype)
    toks = _tokens(cfg["vocab"], 250, 9)
    s = e.alloc_slot()
    outs = [e.step([(s, [t], [0])]) for t in toks]
    assert_close(torch.cat(outs), _plain(e, s, toks, P, cfg, dtype), dtype, "250 tokens one by one")


def test_greedy_generation_through_the_engines_loop(models):
    _, cfg, P = models["B"]
    e = _engine(models, "B", "float32", cache_tokens=8 * 64, n_slots=3)
    prompts = [_tokens(320, n, 70 + n) for n in (5, 63, 1, 120)]
    out = e.generate(prompts, SamplingParams(max_new_tokens=12, temperature=0.0), max_batch=3)
    for p, got in zip(prompts, out):
        assert len(got) == 12
        ctx = list(p)
        for tok in got:
            logits = PL.logits(ctx, P, cfg)[-1]
            want = int(torch.argmax(logits))
            if tok != want:        # only a near tie may differ, and the comparison ends there
                assert float(logits[want] - logits[tok]) <= 2 * TOL["float32"] * float(logits.abs().max())
                break
            ctx.append(tok)
    assert e.cache.slots.n_free == 3


def test_bfloat16_generation_runs_in_a_recorded_decode_session(models):
    e = _engine(models, "B", "bfloat16", cache_tokens=8 * 64, tap=False)
    assert e.graph_safe
    prompts = [_tokens(320, n, n) for n in (9, 40)]
    a = e.generate(prompts, SamplingParams(max_new_tokens=20, temperature=0.0))
    b = e.generate(prompts, SamplingParams(max_new_tokens=20, temperature=0.0))
    assert a == b and all(len(x) == 20 for x in a)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_row_that_stops_early_leaves_the_others_alone(models, dtype):
    """A sequence that meets a stop token becomes a padding row of the decode session; the others
    go on exactly as they do without the stop."""
    e = _engine(models, "B", dtype, cache_tokens=8 * 64, tap=False)
    prompts = [_tokens(320, n, 7 + n) for n in (12, 70, 3)]
    free = e.generate(prompts, SamplingParams(max_new_tokens=16, temperature=0.0))
    stop = free[0][4]
    out = e.generate(prompts, SamplingParams(max_new_tokens=16, temperature=0.0, stop_tokens=[stop]))
    assert len(out[0]) <= 5
    for f, o in zip(free, out):
        cut = f.index(stop) + 1 if stop in f else len(f)
        assert o == f[:cut]
    assert e.cache.slots.n_free == e.cache.n_slots


def test_the_comparison_sees_a_changed_mechanism(models):
    """The tests above would not notice a mechanism that changes nothing: change each in the
    plain implementation and see the engine's logits move away by far more than the tolerance."""
    _, cfg, P = models["A"]
    e = _engine(models, "A", "float32")
    toks = _tokens(211, 60, 2)
    s = e.alloc_slot()
    out = e.step([(s, toks, list(range(60)))]).double().cpu()
    e.free_slot(s)

    def moved(Pmod=None, cfgmod=None):
        ref = PL.logits(toks, Pmod or P, cfgmod or cfg)
        return float((out - ref).abs().max()) / float(ref.abs().max())

    assert moved() <= TOL["float32"]
    no_sink = {k: (torch.full_like(v, -1e4) if k.endswith("mix.sink") else v) for k, v in P.items()}
    assert moved(no_sink) > 1e-3

    def both(c, f):      # layers 1 and 2 are described alike (here by the very same objects)
        f(c["layers"][1])
        if c["layers"][2]["mlp"] is not c["layers"][1]["mlp"]:
            f(c["layers"][2])

    for change in (lambda c: c["layers"][0]["mixer"].update(softcap=4.0),
                   lambda c: c["layers"][0]["mixer"].pop("softcap"),
                   lambda c: c["layers"][0]["mixer"]["rot"].update(dims=12),
                   lambda c: c["layers"][0]["mixer"]["rot"].update(base=41.0),
                   lambda c: c["layers"][0]["mixer"]["mask"].update(size=10),
                   lambda c: c["layers"][0]["mixer"]["mask"].update(size=8),
                   lambda c: c["layers"][0]["mixer"]["mask"].update(keep_first=2),
                   lambda c: c["layers"][0]["mixer"]["mask"].update(keep_first=4),
                   lambda c: c["layers"][0]["mixer"].update(scale=0.31),
                   lambda c: both(c, lambda l: l["mixer"]["mask"].update(size=12)),
                   lambda c: both(c, lambda l: l["mixer"]["mask"].update(size=10)),
                   lambda c: both(c, lambda l: l["mlp"]["router"].update(top=3)),
                   lambda c: both(c, lambda l: l["mlp"]["router"].update(scale=2.4)),
                   lambda c: both(c, lambda l: l["mlp"]["router"]["groups"].update(keep=3)),
                   lambda c: both(c, lambda l: l["mlp"]["router"]["groups"].update(count=2, keep=1)),
                   lambda c: both(c, lambda l: l["mlp"]["expert"].update(limit=1.0)),
                   lambda c: both(c, lambda l: l["mlp"]["shared"].update(limit=0.5)),
                   lambda c: both(c, lambda l: l["mlp"].pop("shared")),
                   lambda c: c["layers"][2].pop("weights_of"),
                   lambda c: c["embedding"]["bigram"].update(mul_prev=8),
                   lambda c: c["embedding"]["bigram"].update(buckets=96),
                   lambda c: c["embedding"].pop("bigram"),
                   lambda c: c["norm"].update(eps=1e-2)):
        other = copy.deepcopy(cfg)
        change(other)
        Pmod = None
        if other["layers"][2].get("weights_of") is None:     # the layer then has tensors of its own
            Pmod = {**P, **{k.replace("l1.", "l2."): v * 0.9 for k, v in P.items() if k.startswith("l1.")}}
        assert moved(Pmod, other) > 1e-4
    for name in ("bigram", "l0.mix.g", "l0.norm1b", "l0.norm2b", "l0.mlp.gate", "l1.mix.q.norm",
                 "l1.mix.k.norm", "l1.mlp.correction", "l1.mlp.router", "l1.mlp.shared.up",
                 "l1.mlp.e3.down", "l3.mix.g", "final.norm", "head"):
        other = dict(P)
        other[name] = P[name] * 0.5 + 0.25
        assert moved(other) > 1e-4, name


def test_trace_replay_as_a_program(models, tmp_path):
    """bin/trace_run as a subprocess on a Lulizen folder: three requests of unequal lengths in one
    batch, decoded together while the shorter ones end, with exactly the tokens they hold as
    --max-tokens."""
    import json
    import subprocess
    from pathlib import Path

    import numpy as np
    folder, cfg, P = models["D"]
    root = Path(__file__).resolve().parent.parent
    V = cfg["vocab"]
    seqs = {"a": _tokens(V, 150, 1), "b": _tokens(V, 70, 2), "c": _tokens(V, 9, 3)}
    heads = {"a": 140, "b": 66, "c": 1}
    steps = [{"step": 0, "entries": [{"id": k, "tokens": seqs[k][:heads[k]], "want": [heads[k] - 1]}
                                     for k in "abc"], "end": []}]
    k = 0
    while True:
        live = [r for r in "abc" if heads[r] + k < len(seqs[r])]
        if not live:
            break
        steps.append({"step": len(steps), "entries": [{"id": r, "tokens": [seqs[r][heads[r] + k]], "want": [0]}
                                                      for r in live],
                      "end": [r for r in live if heads[r] + k + 1 == len(seqs[r])]})
        k += 1
    out = tmp_path / "out"
    proc = subprocess.Popen([str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
                             "--out", str(out), "--max-tokens", str(sum(len(v) for v in seqs.values()))],
                            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, cwd="/")
    for st in steps:
        proc.stdin.write(json.dumps(st) + "\n")
        proc.stdin.flush()
        assert proc.stdout.readline().strip() == f"done {st['step']}"
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0
    refs = {r: PL.logits(seqs[r], P, cfg) for r in "abc"}
    for st in steps:
        got = torch.from_numpy(np.fromfile(out / f"{st['step']}.f32", dtype="<f4").reshape(-1, V))
        want = []
        for e in st["entries"]:
            at = heads[e["id"]] - 1 if st["step"] == 0 else heads[e["id"]] + st["step"] - 1
            want.append(refs[e["id"]][at])
        assert_close(got, torch.stack(want), "float32", f"step {st['step']}")
