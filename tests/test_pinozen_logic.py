"""Pinozen without a GPU: its configuration and weight plan, and the engine's host side (state
rows shared by the two branches of a pair, the paged stores of keys and values, a stretch of
layers that runs several times with storage per run, slots, pages, batches, the generation
loop) on the torch-CPU stand-in of the kernel library, against the plain implementation."""
import copy

import pytest
import torch

import pinozen_models as NM
import plain_pinozen as PN
from nimbus_infer_rs_b200 import Engine, SamplingParams
from nimbus_infer_rs_b200.config import ConfigError, PinozenConfig
from nimbus_infer_rs_b200.config.registry import load_config, resolve_architecture
from nimbus_infer_rs_b200.parts.rotary import rotary_frequencies_by_wavelength
from nimbus_infer_rs_b200.weights.loader import WeightError


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("pinozen")
    return {n: NM.make(root, n) for n in NM.CONFIGS}


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
    assert arch.name == "pinozen" and isinstance(typed, PinozenConfig)
    assert resolve_architecture({"architecture": "pinozen"}).name == "pinozen"
    assert typed.vocab_size == 211 and typed.width == 56 and typed.norm_eps == 3e-5
    assert typed.embedding_scale == 5.0 and typed.logit_scale == 0.5 and typed.max_positions == 320
    a, s = typed.layers[0].mixer.left, typed.layers[0].mixer.right
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.conv, a.softcap) == (4, 2, 12, 20, 3, 8.0)
    assert a.rot.dims == 8 and a.rot.scaling.original == 48 and typed.layers[2].mixer.left.rot.scaling is None
    assert (s.inner, s.state, s.dt_rank, s.conv) == (40, 5, 3, 5)
    assert typed.layers[1].mixer.decay == (0.5, 0.9, 0.99) and typed.layers[1].mlp is None
    assert [i for i, _ in typed.run_order()] == [0, 1, 2, 1, 2, 3]
    assert [f for _, f in typed.run_order()] == [False, True, False, True, False, False]
    assert PinozenConfig.from_json(typed.to_json()) == typed
    # what is left out is absent
    c = PinozenConfig.from_json(NM.CONFIGS["C"])
    assert c.loop is None and c.embedding_scale == 1.0 and c.logit_scale == 1.0
    assert c.layers[0].mixer.left.rot is None and c.layers[0].mixer.left.softcap == 0.0
    assert c.layers[0].mixer.right.conv == 0 and c.layers[2].mixer.left.conv == 0
    # the position table's rows come from the weight file when config.json does not say
    bare = copy.deepcopy(NM.CONFIGS["C"])
    del bare["max_positions"]
    assert PinozenConfig.from_json(bare).with_shapes({"pos": (77, 8)}).max_positions == 77


def test_config_errors_name_every_bad_key():
    bad = copy.deepcopy(NM.CONFIGS["A"])
    bad["layers"][0]["mixer"]["left"]["heads"] = 3            # no multiple of kv_heads
    bad["layers"][0]["mixer"]["left"]["rot"]["dims"] = 14     # more than the head has
    bad["layers"][1]["mixer"]["decay"] = [0.5]                # one per head
    bad["layers"][2]["type"] = "windowed"
    bad["layers"][3]["mlp"] = {"kind": "moe"}
    bad["loop"]["stop"] = 9
    del bad["norm"]
    with pytest.raises(ConfigError) as e:
        PinozenConfig.from_json(bad)
    msg = str(e.value)
    for piece in ("kv_heads", "rot.dims", "decay", "windowed", "moe", "loop", "norm.eps"):
        assert piece in msg, piece


def test_weight_errors_are_listed_together(models, tmp_path):
    _, cfg, tensors = models["C"]
    t = dict(tensors)
    del t["l0.mix.left.sink"]
    t["l2.mix.right.A_log"] = torch.zeros(2, 3)
    t["extra"] = torch.zeros(1)
    folder = NM.write_model(tmp_path / "bad", cfg, t)
    with pytest.raises(WeightError) as e:
        Engine.load(folder, dtype="float32", device="cpu")
    assert e.value.missing == ["l0.mix.left.sink"] and e.value.unexpected == ["extra"]
    assert any("A_log" in w for w in e.value.wrong_shape)


def test_rotary_frequencies_against_the_plain_ones():
    for r in (NM.rot(8, 40.0, (6.0, 1.0, 3.0, 48)), NM.rot(16, 1000.0),
              NM.rot(6, 77.0, (2.0, 2.0, 5.0, 20)), NM.rot(64, 1e6, (8.0, 1.0, 4.0, 8192))):
        f = rotary_frequencies_by_wavelength(r["dims"], r["base"], r.get("scaling"))
        ref = PN.rotary_frequencies(r)
        assert float((f.double() - ref).abs().max()) <= 1e-7 * float(ref.abs().max())
    # all three ranges occur in the first: kept, blended, divided
    f = rotary_frequencies_by_wavelength(8, 40.0, dict(factor=6.0, low=1.0, high=3.0, original=48))
    plain = rotary_frequencies_by_wavelength(8, 40.0, None)
    ratio = (plain / f).tolist()
    assert ratio[0] == 1.0 and 1.0 < ratio[2] < 6.0 and abs(ratio[3] - 6.0) < 1e-5


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompts_and_token_by_token(models, cpu_backend, name):
    _, cfg, P = models[name]
    e = _engine(models, name)
    for n in (1, 2, 37, 80):
        toks = _tokens(cfg["vocab"], n, n)
        ref = PN.logits(toks, P, cfg)
        s = e.alloc_slot()
        _close(e.step([(s, toks, list(range(n)))]), ref)
        e.free_slot(s)
        s = e.alloc_slot()
        one = torch.cat([e.step([(s, [t], [0])]) for t in toks])
        _close(one, ref)
        e.free_slot(s)


def test_layer_by_layer(models, cpu_backend):
    """The stream after every layer run (a layer of the repeated stretch counts each time)."""
    _, cfg, P = models["A"]
    e = _engine(models, "A")
    snaps = []
    for layer in e.model.layers:
        f = layer.block.forward
        layer.block.forward = lambda ctx, x, l, f=f: (f(ctx, x, l), snaps.append(x.clone()))[0]
    toks = _tokens(211, 50, 5)
    s = e.alloc_slot()
    e.step([(s, toks, [0])])
    ref = PN.hidden_states(toks, P, cfg)
    assert len(snaps) == ref.shape[0] == 6
    for got, want in zip(snaps, ref):
        _close(got[:50], want)


def test_portions_down_to_two_tokens(models, cpu_backend):
    """Portions shorter than the convolutions' reach, ending on and beside page ends."""
    _, cfg, P = models["D"]
    e = _engine(models, "D")
    toks = _tokens(99, 150, 3)
    s, at, outs = e.alloc_slot(), 0, []
    for size in (2, 61, 1, 2, 64, 3, 17):
        outs.append(e.step([(s, toks[at:at + size], list(range(size)))]))
        at += size
    _close(torch.cat(outs), PN.logits(toks, P, cfg))


def test_unequal_batch_on_slots_and_pages_used_again(models, cpu_backend):
    """Two batches of unequal prompts decoded together on a cache that holds one batch: the
    second gets the slots, pages and state rows of the first."""
    _, cfg, P = models["A"]
    e = _engine(models, "A", cache_tokens=5 * 64, n_slots=3)
    for round_, lens in enumerate(((100, 5, 66), (1, 90, 30))):
        seqs = [_tokens(211, n, 17 * round_ + i) for i, n in enumerate(lens)]
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
            ref = PN.logits(seqs[i], P, cfg)
            _close(torch.stack(got[i]), ref[heads[i] - 1:])
            e.free_slot(slots[i])
    assert all(g.pool.n_free == g.pool.n_pages for g in e.cache.groups)


def test_every_run_of_a_repeated_layer_has_storage_of_its_own(models, cpu_backend):
    _, cfg, _ = models["A"]
    e = _engine(models, "A")
    kv, st = e.model.storage_requests()
    extra = e.model.extra_storage_requests()
    # six runs: the pair at entry 0 keeps keys and (wider) values in a store each, the pair at
    # entries 2 and 4 keys and values of one size in one store of two planes; every run keeps state
    assert sorted(kv) == [0, 2, 4] and sorted(extra) == [(0, 0)]
    assert sorted(st) == [0, 1, 2, 3, 4, 5]
    assert kv[0].head_dim == 12 and extra[(0, 0)].head_dim == 20 and kv[0].planes == 1
    assert kv[2].head_dim == 16 and kv[2].planes == 2 and kv[4] == kv[2]
    # the pair's row: the attention's last two projected rows, the scan's last four inputs, its state
    assert st[0].n_elements == 2 * (48 + 24 + 40) + 4 * 40 + 40 * 5
    assert st[1].n_elements == 3 * 10 * 14 and st[1] == st[3]
    assert e.cache.state[2].data_ptr() != e.cache.state[4].data_ptr()


def test_state_rows_start_at_zero_for_every_new_sequence(models, cpu_backend):
    _, cfg, P = models["D"]
    e = _engine(models, "D", n_slots=1)
    ref = PN.logits(_tokens(99, 20, 4), P, cfg)
    for _ in range(2):
        s = e.alloc_slot()
        _close(e.step([(s, _tokens(99, 20, 4), list(range(20)))]), ref)
        e.free_slot(s)


def test_the_position_table_bounds_a_sequence(models, cpu_backend):
    e = _engine(models, "C")
    assert e.spec.max_seq_len == 200
    s = e.alloc_slot()
    e.step([(s, _tokens(29, 199, 1), [])])
    e.step([(s, [3], [0])])
    with pytest.raises(Exception):
        e.step([(s, [3], [0])])


def test_greedy_generation_through_the_engines_loop(models, cpu_backend):
    _, cfg, P = models["A"]
    e = _engine(models, "A", cache_tokens=6 * 64, n_slots=3)
    prompts = [_tokens(211, n, 50 + n) for n in (5, 30, 1, 64)]
    out = e.generate(prompts, SamplingParams(max_new_tokens=8, temperature=0.0), max_batch=3)
    for p, got in zip(prompts, out):
        assert len(got) == 8
        ctx = list(p)
        for tok in got:
            logits = PN.logits(ctx, P, cfg)[-1]
            want = int(torch.argmax(logits))
            if tok != want:
                assert float(logits[want] - logits[tok]) <= 1e-4 * float(logits.abs().max())
                break
            ctx.append(tok)
    assert e.cache.slots.n_free == 3


def test_random_weights_mode_and_inspect(cpu_backend):
    cfg = PinozenConfig.from_json(NM.CONFIGS["A"])
    e = Engine.random(cfg, seed=3, dtype="float32", device="cpu", cache_tokens=256)
    s = e.alloc_slot()
    out = e.step([(s, [1, 2, 3], [2])])
    assert out.shape == (1, 211) and torch.isfinite(out).all()
    info = e.inspect()
    assert info["architecture"] == "pinozen" and info["layers"] == 4 and info["tie_head"] is True
    assert e.model.n_params() >= cfg.n_params()       # fused products are filled up with zeros
