"""Lulizen without a GPU: its configuration and weight plan, and the engine's host side (the
previous token in a state row, paged stores that keep a sequence's first pages, layers that run
with another layer's tensors and storage of their own, slots, pages, batches, the generation
loop) on the torch-CPU stand-in of the kernel library, against the plain implementation."""
import copy
import io
import json
import math

import pytest
import torch

import lulizen_models as LM
import plain_lulizen as PL
from nimbus_infer_rs_b200 import Engine, SamplingParams
from nimbus_infer_rs_b200.cache.paged import CacheGroup
from nimbus_infer_rs_b200.config import ConfigError, LulizenConfig
from nimbus_infer_rs_b200.config.registry import load_config, resolve_architecture
from nimbus_infer_rs_b200.parts.base import KVRequest
from nimbus_infer_rs_b200.weights.loader import WeightError


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("lulizen")
    return {n: LM.make(root, n) for n in LM.CONFIGS}


def _tokens(vocab, n, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _close(got, ref, tol=3e-5):
    got, ref = got.double(), ref.double()
    assert got.shape == ref.shape
    assert float((got - ref).abs().max()) <= tol * float(ref.abs().max())


def _engine(models, name, **kw):
    kw.setdefault("cache_tokens", 1024)
    return Engine.load(models[name][0], dtype="float32", device="cpu", **kw)


def test_config_is_read_and_recognised(models):
    folder, cfg, _ = models["A"]
    arch, typed = load_config(folder)
    assert arch.name == "lulizen" and isinstance(typed, LulizenConfig)
    assert resolve_architecture({"architecture": "lulizen"}).name == "lulizen"
    assert typed.vocab_size == 211 and typed.width == 56 and typed.norm_eps == 3e-5
    assert (typed.bigram.buckets, typed.bigram.mul_prev, typed.bigram.mul_cur) == (97, 7, 13)
    a = typed.layers[0].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.softcap, a.mask_size, a.keep_first) == \
        (4, 2, 12, 20, 8.0, 9, 3)
    assert a.rot.dims == 8 and a.rot.base == 40.0
    f = typed.layers[1].mlp
    assert (f.experts, f.top, f.groups, f.keep_groups, f.route_scale) == (6, 2, 3, 2, 2.5)
    assert (f.expert.ff, f.expert.limit, f.shared.ff, f.shared.limit) == (20, 1.5, 24, 0.7)
    assert typed.layers[2].weights_of == 1 and typed.owner(2) == 1 and typed.layers[3].mlp is None
    assert LulizenConfig.from_json(typed.to_json()) == typed
    # what is left out is absent
    c = LulizenConfig.from_json(LM.CONFIGS["C"])
    m = c.layers[0].mixer
    assert c.bigram is None and m.rot is None and m.softcap == 0.0 and m.mask_size == 0
    assert math.isinf(LulizenConfig.from_json(LM.CONFIGS["D"]).layers[0].mlp.expert.limit)
    assert LulizenConfig.from_json(LM.CONFIGS["D"]).layers[0].mlp.correction is False
    # whether a router has a choice bias: the weight file says
    d = LulizenConfig.from_json(LM.CONFIGS["A"])
    assert d.with_shapes({}).layers[1].mlp.correction is False
    assert d.with_shapes({"l1.mlp.correction": (6,)}).layers[2].mlp.correction is True


def test_config_errors_name_every_bad_key():
    bad = copy.deepcopy(LM.CONFIGS["A"])
    bad["layers"][0]["mixer"]["heads"] = 3                     # no multiple of kv_heads
    bad["layers"][0]["mixer"]["rot"]["dims"] = 14              # more than the head has
    bad["layers"][1]["mlp"]["router"]["groups"]["count"] = 4   # six experts in four groups
    bad["layers"][1]["mixer"]["mask"]["keep_first"] = 2        # blocks keep no first tokens
    bad["layers"][3]["type"] = "windowed"
    bad["layers"][0]["mlp"] = {"kind": "sparse"}
    del bad["norm"]
    with pytest.raises(ConfigError) as e:
        LulizenConfig.from_json(bad)
    msg = str(e.value)
    for piece in ("kv_heads", "rot.dims", "groups", "keep_first", "windowed", "sparse", "norm.eps"):
        assert piece in msg, piece
    # a layer that runs with another's tensors is described as that one is
    other = copy.deepcopy(LM.CONFIGS["A"])
    other["layers"][2]["mixer"] = dict(other["layers"][2]["mixer"], softcap=3.0)
    with pytest.raises(ConfigError):
        LulizenConfig.from_json(other)
    circle = copy.deepcopy(LM.CONFIGS["A"])
    circle["layers"][1]["weights_of"] = 2
    with pytest.raises(ConfigError):
        LulizenConfig.from_json(circle)


def test_weight_errors_are_listed_together(models, tmp_path):
    _, cfg, tensors = models["A"]
    t = dict(tensors)
    del t["l1.mix.sink"]
    t["l0.mix.g"] = torch.zeros(2, 3)
    t["l2.norm1"] = torch.zeros(56)          # a layer without tensors of its own has none
    folder = LM.write_model(tmp_path / "bad", cfg, t)
    with pytest.raises(WeightError) as e:
        Engine.load(folder, dtype="float32", device="cpu")
    assert e.value.missing == ["l1.mix.sink"] and e.value.unexpected == ["l2.norm1"]
    assert any("mix.g" in w for w in e.value.wrong_shape)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompts_and_token_by_token(models, cpu_backend, name):
    _, cfg, P = models[name]
    e = _engine(models, name)
    for n in (1, 2, 37, 80):
        toks = _tokens(cfg["vocab"], n, n)
        ref = PL.logits(toks, P, cfg)
        s = e.alloc_slot()
        _close(e.step([(s, toks, list(range(n)))]), ref)
        e.free_slot(s)
        s = e.alloc_slot()
        one = torch.cat([e.step([(s, [t], [0])]) for t in toks])
        _close(one, ref)
        e.free_slot(s)


def test_layer_by_layer(models, cpu_backend):
    """The stream after every layer run (a layer whose tensors run twice counts each time)."""
    _, cfg, P = models["A"]
    e = _engine(models, "A")
    assert e.model.run_order == (0, 1, 1, 2) and len(e.model.layers) == 3
    snaps = []
    for layer in e.model.layers:
        f = layer.block.forward
        layer.block.forward = lambda ctx, x, l, f=f: (f(ctx, x, l), snaps.append(x.clone()))[0]
    toks = _tokens(211, 50, 5)
    s = e.alloc_slot()
    e.step([(s, toks, [0])])
    ref = PL.hidden_states(toks, P, cfg)
    assert len(snaps) == ref.shape[0] == 4
    for got, want in zip(snaps, ref):
        _close(got[:50], want)


@pytest.mark.parametrize("name", ["A", "D"])
def test_portions_down_to_two_tokens(models, cpu_backend, name):
    """Portions that start inside a block, inside a window and right after the kept tokens; the
    token before a portion comes from the state row."""
    _, cfg, P = models[name]
    e = _engine(models, name)
    toks = _tokens(cfg["vocab"], 150, 3)
    s, at, outs = e.alloc_slot(), 0, []
    for size in (2, 61, 1, 2, 64, 3, 17):
        outs.append(e.step([(s, toks[at:at + size], list(range(size)))]))
        at += size
    _close(torch.cat(outs), PL.logits(toks, P, cfg))


def test_unequal_batch_on_slots_and_pages_used_again(models, cpu_backend):
    """Two batches of unequal prompts decoded together on a cache that holds one batch: the
    second gets the slots, pages and state rows of the first."""
    _, cfg, P = models["A"]
    e = _engine(models, "A", cache_tokens=5 * 64, n_slots=3)
    for turn, lens in enumerate(((100, 5, 66), (1, 90, 30))):
        seqs = [_tokens(211, n, 17 * turn + i) for i, n in enumerate(lens)]
        heads = [max(1, n - 3 - i) for i, n in enumerate(lens)]
        slots = [e.alloc_slot() for _ in lens]
        got = {i: [] for i in range(3)}
        out = e.step([(slots[i], seqs[i][:heads[i]], [heads[i] - 1]) for i in range(3)])
        for i in range(3):
            got[i].append(out[i])
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
            ref = PL.logits(seqs[i], P, cfg)
            _close(torch.stack(got[i]), ref[heads[i] - 1:])
            e.free_slot(slots[i])
    assert all(g.pool.n_free == g.pool.n_pages for g in e.cache.groups)


def test_storage_per_run_and_what_each_mask_keeps(models, cpu_backend):
    _, cfg, _ = models["A"]
    e = _engine(models, "A")
    kv, st = e.model.storage_requests()
    extra = e.model.extra_storage_requests()
    # four runs; run 0 keeps keys and (wider) values in a store each; runs 1 and 2 share tensors
    # and keep a store each; the embedding keeps the token before
    assert sorted(kv) == [0, 1, 2, 3] and sorted(extra) == [(0, 0)]
    assert sorted(st) == [-1] and st[-1].n_elements == 1
    assert kv[0] == KVRequest(2, 12, 9, planes=1, keep_first=3)
    assert extra[(0, 0)] == KVRequest(2, 20, 9, planes=1, keep_first=3)
    assert kv[1] == kv[2] == KVRequest(3, 16, 11, planes=2)
    assert e.cache.layer_kv(1).k.data_ptr() != e.cache.layer_kv(2).k.data_ptr()
    assert kv[3] == KVRequest(1, 24, 40, planes=2)


def test_a_window_gives_pages_back_but_not_the_first_ones():
    g = CacheGroup(KVRequest(1, 4, 70, planes=2, keep_first=65), [0], n_pages=12, n_slots=2,
                   max_seq_len=12 * 64, dtype=torch.float32, device="cpu")
    g.ensure(0, 400)
    assert len(g.pages_of(0)) == 7
    assert g.trim(0, 400) == 3                   # pages 2, 3, 4 lie before the window of token 400
    assert g.pages_of(0) == [0, 1, 5, 6]         # the two pages of the first 65 tokens stay
    plain = CacheGroup(KVRequest(1, 4, 70, planes=2), [0], n_pages=12, n_slots=2,
                       max_seq_len=12 * 64, dtype=torch.float32, device="cpu")
    plain.ensure(0, 400)
    assert plain.trim(0, 400) == 5 and plain.pages_of(0) == [5, 6]
    g.release(0)
    assert g.pool.n_free == 12


def test_a_long_sequence_holds_only_what_its_masks_look_back_at(models, cpu_backend):
    """All mixers of B look back at most 128 tokens (plus five kept ones): of a sequence of 700
    tokens, run in portions and then token by token, every store keeps a few pages."""
    _, cfg, P = models["B"]
    e = _engine(models, "B", cache_tokens=11 * 64, n_slots=1)
    toks = _tokens(320, 700, 9)
    ref = PL.logits(toks, P, cfg)
    s, at, outs = e.alloc_slot(), 0, []
    for size in (100, 28, 64, 128, 61, 130, 120, 60):
        outs.append(e.step([(s, toks[at:at + size], list(range(size)))]))
        at += size
    outs += [e.step([(s, [t], [0])]) for t in toks[at:]]
    _close(torch.cat(outs), ref)
    held = sorted(len(g.pages_of(s)) for g in e.cache.groups)
    assert held == [2, 3, 3]        # blocks of 70; blocks of 128; a window of 100 and the first page
    e.free_slot(s)
    assert all(g.pool.n_free == g.pool.n_pages for g in e.cache.groups)


def test_state_rows_do_not_leak_into_a_new_sequence(models, cpu_backend):
    """A slot that is used again: the first token of the new sequence takes the table's last row
    whatever the slot's state row still holds."""
    _, cfg, P = models["D"]
    e = _engine(models, "D", n_slots=1)
    ref = PL.logits(_tokens(99, 20, 4), P, cfg)
    for seed in (8, 4):
        s = e.alloc_slot()
        out = e.step([(s, _tokens(99, 20, seed), list(range(20)))])
        e.free_slot(s)
    _close(out, ref)


def test_greedy_generation_through_the_engines_loop(models, cpu_backend):
    _, cfg, P = models["A"]
    e = _engine(models, "A", cache_tokens=6 * 64, n_slots=3)
    prompts = [_tokens(211, n, 50 + n) for n in (5, 30, 1, 64)]
    out = e.generate(prompts, SamplingParams(max_new_tokens=8, temperature=0.0), max_batch=3)
    for p, got in zip(prompts, out):
        assert len(got) == 8
        ctx = list(p)
        for tok in got:
            logits = PL.logits(ctx, P, cfg)[-1]
            want = int(torch.argmax(logits))
            if tok != want:
                assert float(logits[want] - logits[tok]) <= 1e-4 * float(logits.abs().max())
                break
            ctx.append(tok)
    assert e.cache.slots.n_free == 3


def test_random_weights_mode_and_inspect(cpu_backend):
    cfg = LulizenConfig.from_json(LM.CONFIGS["A"])
    e = Engine.random(cfg, seed=3, dtype="float32", device="cpu", cache_tokens=256)
    s = e.alloc_slot()
    out = e.step([(s, [1, 2, 3], [2])])
    assert out.shape == (1, 211) and torch.isfinite(out).all()
    info = e.inspect()
    assert info["architecture"] == "lulizen" and info["layers"] == 3 and info["tie_head"] is False
    assert e.model.n_params() >= cfg.n_params()       # fused products are filled up with zeros
    small = Engine.random("lulizen-tiny", seed=1, dtype="float32", device="cpu", cache_tokens=256)
    assert small.step([(small.alloc_slot(), [5, 6], [1])]).shape[0] == 1


def test_command_line_and_trace_replay_take_the_design(cpu_backend, tmp_path, monkeypatch, capsys):
    """`random` writes a Lulizen folder that loads again; trace replay drives it with the cache
    the token budget gives, across a portion's start (the token before it is in the state row)."""
    import importlib.machinery
    import importlib.util
    from pathlib import Path

    import numpy as np
    from nimbus_infer_rs_b200.__main__ import main as cli
    folder = tmp_path / "m"
    assert cli(["random", "--preset", "lulizen-tiny", "--out", str(folder), "--seed", "5"]) == 0
    assert json.loads((folder / "config.json").read_text())["architecture"] == "Lulizen"
    capsys.readouterr()
    e = Engine.load(folder, dtype="float32", device="cpu", cache_tokens=128)
    want = e.step([(e.alloc_slot(), [3, 1, 4, 1, 5], [0, 4])])
    path = Path(__file__).resolve().parent.parent / "bin" / "trace_run"
    spec = importlib.util.spec_from_loader("trace_run_cli", importlib.machinery.SourceFileLoader(
        "trace_run_cli", str(path)))
    tr = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(tr)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [3, 1, 4], "want": [0]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [1, 5], "want": [1]}], "end": ["a"]}]
    monkeypatch.setattr("sys.stdin", io.StringIO("".join(json.dumps(s) + "\n" for s in steps)))
    monkeypatch.setattr("sys.argv", ["trace_run", "--model", str(folder), "--dtype", "float32",
                                     "--out", str(tmp_path / "o"), "--max-tokens", "5", "--device", "cpu"])
    assert tr.main() == 0
    assert capsys.readouterr().out.split() == ["done", "0", "done", "1"]
    got = np.concatenate([np.fromfile(tmp_path / "o" / f"{i}.f32", dtype="<f4") for i in (0, 1)])
    _close(torch.from_numpy(got).view(2, -1), want)
