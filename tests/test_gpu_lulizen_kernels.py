"""Lulizen's mechanisms alone on the GPU, each against its plain restatement in float64, with
inputs made so that a fault shows: a query that points at one key (far away, at a page's end,
just inside and just outside a window, a block or the kept first tokens), a sink that takes all
the weight, choice scores below zero beside groups that are left out, a hashed pair across a
portion's start, norms of rows whose mean is far from zero."""
import math

import pytest
import torch

import plain_lulizen as PL
from nimbus_infer_rs_b200.cache import SequenceCache
from nimbus_infer_rs_b200.csrc import ops as ops_mod
from nimbus_infer_rs_b200.csrc.ops import ACT_GELU_TANH, ACT_SWISH_CLAMP
from nimbus_infer_rs_b200.engine.batch import build_layout
from nimbus_infer_rs_b200.parts.base import KVRequest, StateRequest
from nimbus_infer_rs_b200.parts.rotary import rotary_frequencies

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ACT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
DTYPES = ["float32", "bfloat16"]
F64 = torch.float64


@pytest.fixture(scope="module")
def ops():
    return ops_mod.backend()


def _rnd(*shape, seed=0, s=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * s


def _close(got, ref, tol, what=""):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert got.shape == ref.shape, what
    assert torch.isfinite(got).all(), what
    err = float((got - ref).abs().max())
    assert err <= tol * max(float(ref.abs().max()), 1e-30), f"{what}: {err:.3e}"


# ----------------------------------------------------------------------------- row passes
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,d", [(9, 1), (9, 7), (70, 72), (9, 256), (200, 256), (70, 1000), (3, 4100)])
def test_a_centred_norm_added_to_the_stream(ops, dtype, n, d):
    """Rows with a mean far from zero: a norm that does not centre is far off."""
    y, x = _rnd(n, d, seed=1, s=3.0) + 20.0, _rnd(n, d, seed=3) - 5.0
    g, g2 = _rnd(d, seed=4) + 1.0, _rnd(d, seed=6) + 1.0
    x1 = x.double() + PL.layer_norm(y.double(), g.double(), 1e-5)
    for with_next in (False, True):
        xd = x.to(DEV)
        nxt = torch.empty(n, d, device=DEV, dtype=ACT[dtype]) if with_next else None
        cast = torch.empty(n, d, device=DEV, dtype=ACT[dtype]) if with_next else None
        ops.ln_add(y.to(DEV), g.to(DEV), 1e-5, xd, g2.to(DEV) if with_next else None, 3e-4, nxt, cast)
        _close(xd, x1, 3e-6, "stream")
        if with_next:
            _close(nxt, PL.layer_norm(x1, g2.double(), 3e-4), TOL[dtype] / 2, "next norm")
            _close(cast, x1, TOL[dtype] / 4, "rounded stream")


@pytest.mark.parametrize("dtype", DTYPES)
def test_bounded_gate_times_shifted_up(ops, dtype):
    n, d = 13, 37
    x = _rnd(n, 3 + 2 * d + 5, seed=5, s=3.0)
    out = torch.empty(n, d, device=DEV, dtype=ACT[dtype])
    g, u = x[:, 3:3 + d].double(), x[:, 8 + d:8 + 2 * d].double()
    for limit in (0.5, 2.0, math.inf):
        gg, uu = torch.clamp(g, max=limit), torch.clamp(u, -limit, limit)
        ops.glu_rows(x.to(DEV), 3, 8 + d, ACT_SWISH_CLAMP, out, limit)
        _close(out, gg * torch.sigmoid(1.702 * gg) * (uu + 1.0), TOL[dtype] / 2, f"limit {limit}")
    ops.glu_rows(x.to(DEV), 3, 8 + d, ACT_GELU_TANH, out)
    _close(out, PL.gelu_tanh(g) * u, TOL[dtype] / 2, "tanh gelu")


def _layout(pieces, slots, pos0):
    return build_layout([(s, [1] * n, []) for s, n in zip(slots, pieces)], pos0, torch.device(DEV))


@pytest.mark.parametrize("table", ["float32", "bfloat16"])
def test_hashed_pairs_across_portions_and_slots_used_again(ops, table):
    V, D, B, a, b = 50, 24, 13, 31, 17
    wte = _rnd(V, D, seed=1).to(ACT[table])
    pair = _rnd(B + 1, D, seed=2).to(ACT[table])
    last = torch.full((3, 1), 7.0, device=DEV)          # what an earlier sequence left
    seqs = {0: torch.randint(0, V, (40,), generator=torch.Generator().manual_seed(3)).tolist(),
            2: torch.randint(0, V, (11,), generator=torch.Generator().manual_seed(4)).tolist()}
    want = {s: wte[torch.tensor(t)].double() + pair[torch.tensor(PL.hashed_pair_rows(t, B, a, b))].double()
            for s, t in seqs.items()}
    got = {0: [], 2: []}
    at = {0: 0, 2: 0}
    for step in ({0: 5, 2: 1}, {0: 1, 2: 1}, {2: 9}, {0: 33}, {0: 1}):
        entries = [(s, seqs[s][at[s]:at[s] + n], []) for s, n in step.items()]
        lay = build_layout(entries, [at[s] for s in step], torch.device(DEV), pad_rows_to=4)
        out = torch.full((lay.n_rows, D), 9.0, device=DEV)
        ops.embed_hashed(lay, wte.to(DEV), pair.to(DEV), last, out, 1.0, a, b, B)
        r = 0
        for s, n in step.items():
            got[s].append(out[r:r + n].cpu())
            r += n
            at[s] += n
        assert float(out[r:].abs().max() if r < lay.n_rows else 0.0) == 0.0     # padding rows
    for s in seqs:
        _close(torch.cat(got[s]), want[s], 1e-6, f"slot {s}")
    assert last[:, 0].tolist() == [float(seqs[0][-1]), 7.0, float(seqs[2][-1])]


# ----------------------------------------------------------------------------- routing
def _route(ops, z, bias, top, groups, keep, scale):
    n, E = z.shape
    lay = _layout([n], [0], [0])
    idx = torch.empty(n, top, dtype=torch.int32, device=DEV)
    w = torch.empty(n, top, device=DEV)
    ops.moe_route_sigmoid(z.to(DEV), 0, None if bias is None else bias.to(DEV), E, top, groups, keep,
                          2, True, 1e-20, scale, lay, idx, w)
    return idx.cpu().long(), w.cpu()


@pytest.mark.parametrize("E,top,groups,keep", [(12, 3, 4, 2), (6, 2, 3, 2), (8, 3, 4, 2), (9, 4, 3, 2),
                                               (5, 5, 1, 1), (2, 1, 1, 1), (64, 6, 8, 3), (40, 8, 40, 8),
                                               (7, 2, 7, 7)])
def test_choice_among_the_best_groups(ops, E, top, groups, keep):
    z = _rnd(300, E, seed=E, s=2.0)
    for bias in (None, _rnd(E, seed=1, s=0.3), _rnd(E, seed=2, s=0.3) - 3.0):   # the last: all below zero
        idx, w = _route(ops, z, bias, top, groups, keep, 1.5)
        ref_i, ref_w = PL.choose_experts(z.double(), None if bias is None else bias.double(), top,
                                         {"count": groups, "keep": keep} if groups > 1 else None, 1.5)
        assert torch.equal(idx, ref_i)
        _close(w, ref_w, 1e-5, "weights")
        assert float((w.sum(-1) - 1.5).abs().max()) < 1e-4


def test_an_expert_of_a_group_left_out_is_never_taken(ops):
    """Choice scores below zero: were a left-out group's scores counted as 0 instead of as minus
    infinity, its experts would win."""
    E, groups = 8, 4
    z = torch.full((5, E), -1.0)
    z[:, 0:2] = 3.0                      # group 0 is best, group 1 second by a little
    z[:, 2] = -0.9
    bias = torch.full((E,), -2.0)        # every choice score is negative
    idx, w = _route(ops, z, bias, 3, groups, 2, 1.0)
    assert set(idx[0].tolist()) == {0, 1, 2}
    # equal scores: the lower group, the lower expert
    idx, _ = _route(ops, torch.zeros(4, E), None, 2, groups, 1, 1.0)
    assert idx.tolist() == [[0, 1]] * 4
    # a row of padding chooses nothing
    lay = build_layout([(0, [1, 1], [])], [0], torch.device(DEV), pad_rows_to=4)
    idx = torch.zeros(4, 2, dtype=torch.int32, device=DEV)
    w = torch.ones(4, 2, device=DEV)
    ops.moe_route_sigmoid(torch.zeros(4, E, device=DEV), 0, None, E, 2, 1, 1, 2, True, 0.0, 1.0, lay, idx, w)
    assert idx[2:].tolist() == [[-1, -1]] * 2 and float(w[2:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,D,E,F,top", [(5, 56, 6, 20, 2), (300, 64, 4, 48, 2), (1500, 128, 8, 64, 3)])
def test_experts_with_bounded_halves(ops, dtype, n, D, E, F, top):
    """The three products that run the experts' first halves (CUDA cores, mma.sync, tcgen05 from
    1024 pairs on) with the bounded combiner, against one expert at a time."""
    x = _rnd(n, D, seed=1).to(ACT[dtype])
    gate = (_rnd(E, F, D, seed=2) * (2.0 / math.sqrt(D))).to(ACT[dtype])
    up = (_rnd(E, F, D, seed=3) * (2.0 / math.sqrt(D))).to(ACT[dtype])
    idx = torch.stack([torch.randperm(E, generator=torch.Generator().manual_seed(i))[:top] for i in range(n)])
    offsets = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    order = torch.empty(n * top, dtype=torch.int32, device=DEV)
    place = torch.empty(n * top, dtype=torch.int32, device=DEV)
    ops.moe_group(idx.to(torch.int32).to(DEV), E, offsets, order, place)
    mid = torch.empty(n * top, F, device=DEV, dtype=ACT[dtype])
    limit = 0.8
    ops.moe_linear(x.to(DEV), order, top, offsets, gate.to(DEV), up.to(DEV), mid, ACT_SWISH_CLAMP, limit)
    pl = place.cpu().view(n, top)
    ref = torch.zeros(n * top, F, dtype=F64)
    for r in range(n):
        for k in range(top):
            e = int(idx[r, k])
            g = torch.clamp(gate[e].double() @ x[r].double(), max=limit)
            u = torch.clamp(up[e].double() @ x[r].double(), -limit, limit)
            ref[pl[r, k]] = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    _close(mid, ref, TOL[dtype], "first halves")


# ----------------------------------------------------------------------------- attention
def _stores(dtype, G, d, dv, tokens, window=0, keep_first=0, fill=None):
    shared = d == dv
    cache = SequenceCache({0: KVRequest(G, d, window, 2 if shared else 1, keep_first=keep_first)}, {},
                          cache_tokens=tokens, max_seq_len=tokens, dtype=ACT[dtype],
                          device=torch.device(DEV), n_slots=4,
                          extra_kv_requests={} if shared else
                          {(0, 0): KVRequest(G, dv, window, 1, keep_first=keep_first)})
    if fill is not None:           # what an earlier owner of the pages left behind
        for g in cache.groups:
            g.storage.fill_(fill)
    return cache


def _plain(q, k, v, kind, mask, rot, norms, scale, cap, sink, gate):
    q, k, v = q.double(), k.double(), v.double()
    if norms is not None:
        q, k = PL.rms_unit(q, norms[0].double(), 1e-5), PL.rms_unit(k, norms[1].double(), 1e-5)
    if rot:
        q, k = PL.rotate_halves(q, *rot), PL.rotate_halves(k, *rot)
    o = PL.attend(q, k, v, PL.visible(q.shape[0], kind, mask), scale, cap,
                  None if sink is None else sink.double())
    if gate is not None:
        o = o * torch.sigmoid(gate.double())[:, :, None]
    return o.reshape(q.shape[0], -1)


def _attention(ops, dtype, q, k, v, pieces, kind="attention_2", mask=None, rot=None, norms=None,
               scale=1.0, cap=0.0, sink=None, gate=None, fill=None, trim=False):
    """Norm + rotation + append, then attention, over one sequence cut into ``pieces``.
    q [T, H, d], k [T, G, d], v [T, G, dv]: projected rows (fp32)."""
    T, H, d = q.shape
    G, dv = k.shape[1], v.shape[2]
    window = keep = chunk = 0
    if mask:
        if kind == "attention":
            chunk = mask["size"]
        else:
            window, keep = mask["size"], mask.get("keep_first", 0)
    cache = _stores(dtype, G, d, dv, T + 64, (window or chunk) if trim else 0, keep if trim else 0, fill)
    freq = rotary_frequencies(rot[0], rot[1])[0].to(DEV) if rot else None
    cols = [q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)]
    if gate is not None:
        cols.append(gate)
    fused = torch.cat(cols, dim=1)
    pad = -fused.shape[1] % 8
    fused = torch.cat([fused, torch.zeros(T, pad)], dim=1).to(DEV)
    keys = cache.layer_kv(0)
    values = keys if d == dv else cache.layer_kv((0, 0))
    slot = cache.alloc_slot()
    outs, at = [], 0
    for n in pieces:
        cache.reserve([(slot, n)])
        lay = build_layout([(slot, [1] * n, [])], [at], torch.device(DEV))
        rows = fused[at:at + n].contiguous()
        qo = torch.empty(n, H * d, device=DEV, dtype=ACT[dtype])
        ops.qkv_norm_rope_append(rows, 0, H * d, H * d + G * d,
                                 None if norms is None else norms[0].to(DEV),
                                 None if norms is None else norms[1].to(DEV), 1e-5, freq,
                                 rot[0] if rot else 0, 1.0, lay, keys, values, H, dv, qo, True)
        out = torch.empty(n, H * dv, device=DEV, dtype=ACT[dtype])
        ops.attention_masked(qo, lay, keys, values, H, None if sink is None else sink.to(DEV), out,
                             scale, cap, window, keep, chunk, rows if gate is not None else None,
                             H * d + G * d + G * dv)
        cache.advance(slot, n)
        outs.append(out.float().cpu())
        at += n
    ops.raise_device_errors()
    return torch.cat(outs)


SHAPES = [  # H, G, d, dv, kind, mask, rot, norms, cap, sink, gate
    (4, 2, 12, 20, "attention_2", {"size": 9, "keep_first": 3}, (8, 40.0), False, 8.0, False, True),
    (3, 3, 16, 16, "attention", {"size": 11}, (16, 1000.0), True, 30.0, True, False),
    (4, 2, 64, 64, "attention_2", {"size": 100, "keep_first": 5}, (32, 1e4), False, 20.0, False, True),
    (8, 2, 64, 64, "attention", {"size": 70}, (64, 1e6), True, 15.0, True, False),
    (6, 3, 128, 128, "attention_2", {"size": 90, "keep_first": 6}, (32, 4e4), False, 45.0, False, True),
    (2, 1, 128, 128, "attention", {"size": 128}, (64, 1e5), True, 0.0, True, False),
    (4, 4, 32, 32, "attention", {"size": 64}, (32, 500.0), True, 15.0, True, False),
    (16, 4, 128, 128, "attention_2", {"size": 130, "keep_first": 70}, (128, 1e4), False, 30.0, False, True),
    (5, 5, 7, 9, "attention_2", {"size": 3, "keep_first": 10}, (4, 20.0), False, 0.0, False, True),
    (6, 2, 10, 6, "attention", {"size": 1}, (6, 77.0), True, 5.0, True, False),
    (1, 1, 2, 2, "attention", None, None, True, 0.0, True, False),
    (2, 1, 48, 48, "attention_2", None, (48, 100.0), False, 4.0, True, True),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", range(len(SHAPES)))
def test_attention_whole_in_portions_and_token_by_token(ops, dtype, shape):
    H, G, d, dv, kind, mask, rot, norm, cap, sink, gate = SHAPES[shape]
    T = 203
    q, k, v = _rnd(T, H, d, seed=1), _rnd(T, G, d, seed=2), _rnd(T, G, dv, seed=3)
    norms = (_rnd(d, seed=4, s=0.2) + 1.0, _rnd(d, seed=5, s=0.2) + 1.0) if norm else None
    sinks = _rnd(H, seed=6, s=1.5) if sink else None
    gates = _rnd(T, H, seed=7, s=2.0) if gate else None
    scale = 1.0 / math.sqrt(d) if norms is None else 4.0 / d
    tol = TOL[dtype]
    ref = _plain(q, k, v, kind, mask, rot, norms, scale, cap, sinks, gates)
    kw = dict(kind=kind, mask=mask, rot=rot, norms=norms, scale=scale, cap=cap, sink=sinks, gate=gates)
    for pieces, trim in (((T,), False), ((2, 61, 1, 2, 64, 3, 70), True), ((130,) + (1,) * 73, True)):
        got = _attention(ops, dtype, q, k, v, pieces, fill=float("nan"), trim=trim, **kw)
        _close(got, ref, tol, f"shape {shape} in pieces {pieces[:3]}")
    if dtype == "bfloat16" and d == dv and d in (64, 128):
        # the same heads on the mma.sync prompt kernel, which takes them when tcgen05 is off
        ops.use_tcgen05 = False
        try:
            got = _attention(ops, dtype, q, k, v, (2, 61, 1, 2, 64, 3, 70), fill=float("nan"), trim=True, **kw)
        finally:
            ops.use_tcgen05 = True
        _close(got, ref, tol, f"shape {shape} without tcgen05")


def _pointed(T, H, G, d, dv, at, to, seed=0):
    """Queries and keys of small random numbers, except that the query at position ``at`` and the
    key at position ``to`` share one large direction: that score stands out from all others.
    The first number of a value is 1 at position ``to`` and 0 elsewhere, so the first number of
    the result is the weight that key got; the second number names the position."""
    q, k = _rnd(T, H, d, seed=seed, s=0.05), _rnd(T, G, d, seed=seed + 1, s=0.05)
    v = torch.zeros(T, G, dv)
    v[to, :, 0] = 1.0
    v[:, :, 1] = torch.arange(T, dtype=torch.float32)[:, None]
    q[at, :, -1] += 6.0
    k[to, :, -1] += 6.0
    return q, k, v


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [16, 64, 128])
def test_a_key_just_inside_and_just_outside(ops, dtype, d):
    """One query, one key that would take nearly all the weight: it does when it is seen, and
    gets none when it is one token beyond the edge.  Windows, kept
    first tokens and blocks; in a prompt, across portions and in one-token steps; edges on and
    beside page ends."""
    H, G, T = 2, 1, 330
    scale = 1.0
    cases = []
    for size, keep in ((80, 6), (64, 0), (65, 64), (130, 1)):
        mask = {"size": size, "keep_first": keep}
        for at in (T - 3, 200, 129):
            cases += [("attention_2", mask, at, at - size + 1, True), ("attention_2", mask, at, at - size, False)]
            if keep:
                cases += [("attention_2", mask, at, keep - 1, True), ("attention_2", mask, at, keep, at - keep < size)]
    for size in (64, 70, 128, 190):
        mask = {"size": size}
        for at in (T - 3, 2 * size + 5, 2 * size):
            if at >= T - 2:
                continue
            first = (at // size) * size
            cases += [("attention", mask, at, first, True), ("attention", mask, at, first - 1, False)]
    cases += [("attention_2", None, T - 3, 0, True), ("attention_2", None, T - 3, 63, True)]
    for kind, mask, at, to, seen in cases:
        if to < 0:
            continue
        q, k, v = _pointed(T, H, G, d, d, at, to, seed=at + to)
        sink = torch.zeros(H) if kind == "attention" else None
        # whole; the query decoded alone after a prompt that ends two tokens before it; a cut
        # between the key and the query
        for pieces in ((T,), (at - 2, 1, 1, 1, 1, T - at - 2), (to + 1, T - to - 1)):
            if sum(pieces) != T or min(pieces) < 1:
                continue
            got = _attention(ops, dtype, q, k, v, pieces, kind=kind, mask=mask, scale=scale, sink=sink,
                             trim=True)
            weight = float(got[at, 0])
            if seen:
                assert weight > 0.97, (kind, mask, at, to, pieces[:3], weight)
            else:
                assert weight == 0.0, (kind, mask, at, to, pieces[:3], weight)
        _close(_attention(ops, dtype, q, k, v, (T,), kind=kind, mask=mask, scale=scale, sink=sink),
               _plain(q, k, v, kind, mask, None, None, scale, 0.0, sink, None), TOL[dtype], "whole")


@pytest.mark.parametrize("dtype", DTYPES)
def test_sinks_caps_and_the_first_token(ops, dtype):
    H, G, d, T = 4, 2, 32, 90
    # numbers that bfloat16 holds exactly: scores near zero, where the cap bends most, are then
    # the same numbers in both precisions
    q, k, v = (_rnd(T, n, d, seed=i).bfloat16().float() for i, n in ((1, H), (2, G), (3, G)))
    mask = {"size": 40}
    # a sink of +40 takes all the weight, one of -40 none
    out = _attention(ops, dtype, q, k, v, (T,), kind="attention", mask=mask, scale=0.2,
                     sink=torch.full((H,), 40.0))
    assert float(out.abs().max()) < 1e-6
    for s in (-40.0, 0.0, 3.0):
        sink = torch.full((H,), s)
        _close(_attention(ops, dtype, q, k, v, (T,), kind="attention", mask=mask, scale=0.2, sink=sink),
               _plain(q, k, v, "attention", mask, None, None, 0.2, 0.0, sink, None), TOL[dtype], f"sink {s}")
    # scores far beyond the cap: all keys weigh the same, and the sink (not capped) still counts
    sink = torch.full((H,), 5.0)
    big = _attention(ops, dtype, q * 64, k, v, (T,), kind="attention", mask=mask, scale=1.0, cap=2.0, sink=sink)
    _close(big, _plain(q * 64, k, v, "attention", mask, None, None, 1.0, 2.0, sink, None), TOL[dtype], "cap")
    # the first token alone sees itself (and the sink)
    one = _attention(ops, dtype, q[:1], k[:1], v[:1], (1,), kind="attention", mask=mask, scale=0.2,
                     sink=torch.zeros(H))
    _close(one, _plain(q[:1], k[:1], v[:1], "attention", mask, None, None, 0.2, 0.0, torch.zeros(H), None),
           TOL[dtype], "first token")


@pytest.mark.parametrize("dtype", DTYPES)
def test_an_unequal_batch_against_each_alone(ops, dtype):
    """Three sequences of unequal lengths in one step, then decoded together: every row as when
    its sequence runs alone."""
    H, G, d = 4, 2, 64
    mask = {"size": 70, "keep_first": 3}
    lens, heads = (150, 9, 70), (140, 1, 66)
    cache = _stores(dtype, G, d, d, 6 * 64)
    keys = cache.layer_kv(0)
    freq = rotary_frequencies(32, 1e4)[0].to(DEV)
    data = [(_rnd(n, H, d, seed=10 + i), _rnd(n, G, d, seed=20 + i), _rnd(n, G, d, seed=30 + i),
             _rnd(n, H, seed=40 + i)) for i, n in enumerate(lens)]
    fused = [torch.cat([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1), g], 1).to(DEV)
             for (q, k, v, g), n in zip(data, lens)]
    slots = [cache.alloc_slot() for _ in lens]
    got = [[] for _ in lens]

    def step(parts):      # parts: (sequence, start, count)
        cache.reserve([(slots[i], n) for i, _, n in parts])
        lay = build_layout([(slots[i], [1] * n, []) for i, _, n in parts], [a for _, a, _ in parts],
                           torch.device(DEV), pad_rows_to=8)
        rows = torch.zeros(lay.n_rows, fused[0].shape[1], device=DEV)
        r = 0
        for i, a, n in parts:
            rows[r:r + n] = fused[i][a:a + n]
            r += n
        qo = torch.empty(lay.n_rows, H * d, device=DEV, dtype=ACT[dtype])
        ops.qkv_norm_rope_append(rows, 0, H * d, H * d + G * d, None, None, 0.0, freq, 32, 1.0, lay, keys,
                                 keys, H, d, qo, True)
        out = torch.empty(lay.n_rows, H * d, device=DEV, dtype=ACT[dtype])
        ops.attention_masked(qo, lay, keys, keys, H, None, out, 0.125, 10.0, 70, 3, 0, rows,
                             H * d + 2 * G * d)
        r = 0
        for i, a, n in parts:
            got[i].append(out[r:r + n].float().cpu())
            cache.advance(slots[i], n)
            r += n

    step([(i, 0, h) for i, h in enumerate(heads)])
    k = 0
    while True:
        live = [(i, heads[i] + k, 1) for i in range(3) if heads[i] + k < lens[i]]
        if not live:
            break
        step(live)
        k += 1
    for i, (q, kk, v, g) in enumerate(data):
        ref = _plain(q, kk, v, "attention_2", mask, (32, 1e4), None, 0.125, 10.0, None, g)
        _close(torch.cat(got[i]), ref, TOL[dtype], f"sequence {i}")
