"""Pinozen's mechanisms alone on the GPU, each against its plain restatement in float64, with
inputs made so that a fault shows: a query that points at one far key among hundreds, scores
that the cap bends, a sink that takes all the weight, recurrences that have to remember their
first token, convolutions across portion and page ends, state rows used again."""
import math

import pytest
import torch

import plain_pinozen as PN
from nimbus_infer_rs_b200.cache import SequenceCache
from nimbus_infer_rs_b200.csrc import ops as ops_mod
from nimbus_infer_rs_b200.csrc.ops import ACT_GELU_TANH, ACT_NONE, ACT_RELU, ACT_RELU2, ACT_SILU
from nimbus_infer_rs_b200.engine.batch import build_layout
from nimbus_infer_rs_b200.parts.base import KVRequest, StateRequest
from nimbus_infer_rs_b200.parts.rotary import rotary_frequencies_by_wavelength

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ACT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


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
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d", [1, 7, 72, 256, 1000, 4100])
def test_two_normed_results_averaged_into_the_stream(ops, dtype, d):
    n = 9
    a, b, x = _rnd(n, d, seed=1, s=3.0), _rnd(n, d, seed=2, s=0.01), _rnd(n, d, seed=3)
    ga, gb, g2 = _rnd(d, seed=4) + 1.0, _rnd(d, seed=5) + 1.0, _rnd(d, seed=6) + 1.0
    x1 = x.double() + 0.5 * (PN.rms_norm(a.double(), ga.double(), 1e-5)
                             + PN.rms_norm(b.double(), gb.double(), 1e-5))
    for with_next in (False, True):
        xd = x.to(DEV)
        nxt = torch.empty(n, d, device=DEV, dtype=ACT[dtype]) if with_next else None
        ops.rms_pair_add(a.to(DEV), ga.to(DEV), b.to(DEV), gb.to(DEV), 1e-5, 0.5, xd,
                         g2.to(DEV) if with_next else None, 3e-4, nxt)
        _close(xd, x1, 2e-6, "stream")
        if with_next:
            _close(nxt, PN.rms_norm(x1, g2.double(), 3e-4), TOL[dtype] / 2, "next norm")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gates_casts_and_the_gated_norm(ops, dtype):
    n, d = 13, 37
    x = _rnd(n, 3 + 2 * d + 5, seed=5, s=3.0)
    xd = x.to(DEV)
    out = torch.empty(n, d, device=DEV, dtype=ACT[dtype])
    g, u = x[:, 3:3 + d].double(), x[:, 8 + d:8 + 2 * d].double()
    for act, f in ((ACT_RELU, torch.relu), (ACT_SILU, PN.silu), (ACT_NONE, lambda z: z),
                   (ACT_RELU2, lambda z: torch.relu(z) ** 2),
                   (ACT_GELU_TANH, lambda z: 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))))):
        ops.glu_rows(xd, 3, 8 + d, act, out)
        _close(out, f(g) * u, TOL[dtype] / 2, f"gate with activation {act}")
    wide = torch.full((n, 2 * d + 3), 7.0, device=DEV, dtype=ACT[dtype])
    src = _rnd(n, d, seed=6)
    ops.cast_cols(src.to(DEV), wide, d + 1)
    _close(wide[:, d + 1:2 * d + 1], src, TOL[dtype] / 4, "columns written")
    assert bool((wide[:, :d + 1] == 7.0).all()) and bool((wide[:, 2 * d + 1:] == 7.0).all())
    gamma = _rnd(d, seed=7) + 1.0
    rows = _rnd(n, d, seed=8, s=5.0)
    ops.rmsnorm_gated(rows.to(DEV), gamma.to(DEV), xd, 8 + d, 1e-4, out)
    _close(out, PN.rms_norm(rows.double(), gamma.double(), 1e-4) * torch.sigmoid(u), TOL[dtype] / 2,
           "norm times gate")


# ----------------------------------------------------------------------------- storage helpers
def _stores(dtype, G, d, dv, n_state, tokens, n_slots=None, fill=None):
    """Keys and values of one size share a store of two planes, as in the part; else a store each."""
    shared = d == dv
    cache = SequenceCache({0: KVRequest(G, d, 0, 2 if shared else 1)},
                          {0: StateRequest(n_state)} if n_state else {},
                          cache_tokens=tokens, max_seq_len=tokens, dtype=ACT[dtype],
                          device=torch.device(DEV), n_slots=n_slots,
                          extra_kv_requests={} if shared else {(0, 0): KVRequest(G, dv, 0, 1)})
    if fill is not None:           # what an earlier owner of the pages left behind
        for g in cache.groups:
            g.storage.fill_(fill)
    return cache


def _attention(ops, dtype, q, k, v, conv, rot, scale, softcap, sink, pieces, fill=None):
    """Convolution + rotation + append, then attention, over one sequence cut into ``pieces``.
    q [T, H, d], k [T, G, d], v [T, G, dv]: projected rows (fp32); conv: [channels, taps] or None."""
    T, H, d = q.shape
    G, dv = k.shape[1], v.shape[2]
    C = H * d + G * d + G * dv
    taps = 0 if conv is None else conv.shape[1]
    cache = _stores(dtype, G, d, dv, max(taps - 1, 0) * C, T + 64, fill=fill)
    freq, dims = None, 0
    if rot:
        dims = rot["dims"]
        freq = rotary_frequencies_by_wavelength(dims, rot["base"], rot.get("scaling")).to(DEV)
    fused = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1).to(DEV)
    w = None if conv is None else conv.to(DEV).contiguous()
    slot, at, outs = cache.alloc_slot(), 0, []
    for n in pieces:
        cache.reserve([(slot, n)])
        lay = build_layout([(slot, [0] * n, [])], [at], DEV)
        keys = cache.layer_kv(0)
        values = keys if d == dv else cache.layer_kv_extra(0)[0]
        qo = torch.empty(n, H * d, device=DEV, dtype=ACT[dtype])
        ops.conv_rope_append(fused[at:at + n].contiguous(), 0, w, taps, cache.layer_state(0), freq, dims,
                             lay, keys, values, H, dv, qo)
        out = torch.empty(n, H * dv, device=DEV, dtype=ACT[dtype])
        ops.attention_capped(qo, lay, keys, values, H, None if sink is None else sink.to(DEV), out,
                             scale, softcap)
        outs.append(out.float().cpu())
        cache.advance(slot, n)
        at += n
    assert at == T
    return torch.cat(outs).view(T, H, dv)


def _plain_attention(q, k, v, conv, rot, scale, softcap, sink):
    T, H, d = q.shape
    G, dv = k.shape[1], v.shape[2]
    q, k, v = q.double().reshape(T, -1), k.double().reshape(T, -1), v.double().reshape(T, -1)
    if conv is not None:
        c = conv.double()
        q = PN.causal_conv(q, c[:H * d])
        k = PN.causal_conv(k, c[H * d:H * d + G * d])
        v = PN.causal_conv(v, c[H * d + G * d:])
    pos = torch.arange(T)
    q = PN.rotate_interleaved(q.view(T, H, d), pos, rot)
    k = PN.rotate_interleaved(k.view(T, G, d), pos, rot)
    return PN.capped_sink_attention(q, k, v.view(T, G, dv), scale, softcap,
                                    None if sink is None else sink.double())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", [
    dict(H=4, G=2, d=12, dv=20, taps=3, cap=8.0, rot=dict(dims=8, base=40.0, scaling=dict(factor=6.0, low=1.0, high=3.0, original=48))),
    dict(H=3, G=3, d=16, dv=16, taps=4, cap=30.0, rot=dict(dims=16, base=1000.0)),
    dict(H=6, G=2, d=10, dv=6, taps=2, cap=5.0, rot=dict(dims=6, base=77.0)),
    dict(H=1, G=1, d=2, dv=2, taps=1, cap=0.0, rot=None),
    dict(H=2, G=1, d=3, dv=1, taps=0, cap=2.0, rot=dict(dims=2, base=10.0)),
    dict(H=4, G=1, d=64, dv=64, taps=4, cap=0.0, scale=0.04, rot=dict(dims=64, base=1e4)),
    dict(H=2, G=2, d=33, dv=130, taps=7, cap=50.0, rot=dict(dims=32, base=500.0, scaling=dict(factor=4.0, low=1.0, high=4.0, original=64))),
    # an odd head size: the second head's rotated pairs start at odd channels, and one of them
    # lies across the border between two blocks of 128 channels
    dict(H=2, G=1, d=85, dv=9, taps=3, cap=9.0, scale=0.1, rot=dict(dims=84, base=200.0)),
    # head sizes that the tensor-core prompt kernel and the decode kernel of plain attention take
    dict(H=6, G=2, d=64, dv=64, taps=3, cap=4.0, scale=0.09, rot=dict(dims=32, base=300.0)),
    dict(H=4, G=4, d=128, dv=128, taps=2, cap=12.0, scale=0.05, rot=dict(dims=128, base=1e4)),
    dict(H=8, G=1, d=128, dv=128, taps=0, cap=0.0, scale=0.06, rot=None),
    dict(H=2, G=1, d=64, dv=128, taps=4, cap=6.0, scale=0.1, rot=dict(dims=64, base=1e3)),
])
def test_attention_whole_in_portions_and_token_by_token(ops, dtype, case):
    T, H, G, d, dv = 200, case["H"], case["G"], case["d"], case["dv"]
    q, k, v = _rnd(T, H, d, seed=1, s=2.0), _rnd(T, G, d, seed=2, s=2.0), _rnd(T, G, dv, seed=3)
    conv = _rnd(H * d + G * d + G * dv, case["taps"], seed=4, s=0.7) if case["taps"] else None
    sink = _rnd(H, seed=5, s=1.5)
    args = (conv, case["rot"], case.get("scale", 0.3), case["cap"], sink)
    ref = _plain_attention(q, k, v, *args)
    for pieces in ([T], [2, 61, 1, 2, 64, 3, 67], [60] + [1] * 140):
        got = _attention(ops, dtype, q, k, v, *args, pieces, fill=float("nan"))
        _close(got, ref, TOL[dtype], f"{case} in {len(pieces)} pieces")


@pytest.mark.parametrize("d,dv", [(16, 8), (64, 64)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_query_that_points_at_one_far_key(ops, dtype, d, dv):
    """700 tokens; every query points along one direction that only one key, far back and just
    before a page's end, shares: its value carries nearly all the weight at every later
    position, in a prompt, across a portion's start and decoded alone."""
    T, far = 700, 63
    a = torch.zeros(d)
    a[3] = 1.0
    k = _rnd(T, 1, d, seed=9)
    k[:, 0, 3] = 0.0                         # everyone else is orthogonal to `a`
    k[far, 0] = a * 4.0
    v = _rnd(T, 1, dv, seed=10)
    q = (a * 5.0).repeat(T, 2, 1)
    ref = _plain_attention(q, k, v, None, None, 1.0, 0.0, None)
    assert float((ref[far + 200, 0] - v[far, 0].double()).abs().max()) < 1e-4    # it stands out
    for pieces in ([T], [63, 1, 1, 635], [300] + [1] * 400):
        got = _attention(ops, dtype, q, k, v, None, None, 1.0, 0.0, None, pieces)
        _close(got, ref, TOL[dtype], f"far key in {len(pieces)} pieces")
    # with a cap the far key's score is bent down to the cap and its lead shrinks
    capped = _plain_attention(q, k, v, None, None, 1.0, 3.0, None)
    assert float((capped[far + 200, 0] - ref[far + 200, 0]).abs().max()) > 1e-2
    got = _attention(ops, dtype, q, k, v, None, None, 1.0, 3.0, None, [300] + [1] * 400)
    _close(got, capped, TOL[dtype], "far key under a cap")


@pytest.mark.parametrize("d", [8, 64, 128])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_a_sink_that_takes_everything(ops, dtype, d):
    T, H = 70, 2
    # exact in bfloat16, so that the cap's steep middle does not magnify the inputs' rounding
    q, k, v = (_rnd(T, n, d, seed=i).bfloat16().float() for i, n in ((1, H), (2, 1), (3, 1)))
    big = torch.tensor([40.0, -40.0])
    scale = 0.5 * math.sqrt(8 / d)
    ref = _plain_attention(q, k, v, None, None, scale, 0.0, big)
    assert float(ref[:, 0].abs().max()) < 1e-10 and float(ref[:, 1].abs().max()) > 0.1
    for pieces in ([T], [1] * T):
        got = _attention(ops, dtype, q, k, v, None, None, scale, 0.0, big, pieces)
        _close(got, ref, TOL[dtype], "a sink of +40 and one of -40")
    # the sink is neither scaled nor capped: under a cap of 1 a sink of 3 still outweighs a key
    small = torch.tensor([3.0, 3.0])
    ref = _plain_attention(q * 64, k, v, None, None, scale, 1.0, small)
    assert float((ref - _plain_attention(q * 64, k, v, None, None, scale, 1.0, small * 0)).abs().max()) > 0.05
    for pieces in ([3, 67], [1] * T):
        got = _attention(ops, dtype, q * 64, k, v, None, None, scale, 1.0, small, pieces)
        _close(got, ref, TOL[dtype], "sink beside capped scores")
    first = _plain_attention(q[:1] * 64, k[:1], v[:1], None, None, scale, 1.0, small)
    _close(got[:1], first, TOL[dtype], "the first token sees itself and the sink")


# ----------------------------------------------------------------------------- convolution alone
@pytest.mark.parametrize("taps", [1, 2, 4, 9])
def test_convolution_with_bias_and_activation_in_portions(ops, taps):
    T, C = 150, 50
    u, w, b = _rnd(T, 3 + C, seed=1), _rnd(C, taps, seed=2, s=0.7), _rnd(C, seed=3)
    ref = PN.silu(PN.causal_conv(u[:, 3:].double(), w.double(), b.double()))
    for pieces in ([T], [2, 61, 1, 2, 64, 3, 17], [1] * T):
        cache = _stores("float32", 1, 1, 1, max(taps - 1, 0) * C, 256, n_slots=2)
        cache.alloc_slot()                         # the sequence gets the second slot's row
        slot, at, outs = cache.alloc_slot(), 0, []
        for n in pieces:
            cache.reserve([(slot, n)])
            lay = build_layout([(slot, [0] * n, [])], [at], DEV)
            out = torch.empty(n, C, device=DEV)
            half = torch.empty(n, C, device=DEV, dtype=torch.bfloat16)
            ops.conv_act(u[at:at + n].to(DEV).contiguous(), 3, w.to(DEV), b.to(DEV), taps, ACT_SILU,
                         cache.layer_state(0), lay, out, half)
            _close(half, out, 5e-3, "rounded copy")
            outs.append(out.cpu())
            cache.advance(slot, n)
            at += n
        _close(torch.cat(outs), ref, 2e-6, f"{taps} taps in {len(pieces)} pieces")
        if taps > 1:       # the state row holds the last inputs, oldest first; the other row is untouched
            want = u[T - (taps - 1):, 3:].reshape(-1)
            _close(cache.layer_state(0)[slot].cpu(), want, 1e-7, "state after the sequence")
            assert float(cache.layer_state(0)[1 - slot].abs().max()) == 0.0


# ----------------------------------------------------------------------------- selective scan
def _scan(ops, dtype, x, low, dt_lin, z, dt_bias, a_log, d_skip, R, N, pieces):
    T, inner = x.shape
    cache = _stores("float32", 1, 1, 1, inner * N, 64)
    slot, at, outs = cache.alloc_slot(), 0, []
    zz = torch.cat([_rnd(T, 5, seed=99), z], dim=1).to(DEV)        # the gates sit at column 5
    for n in pieces:
        cache.reserve([(slot, 0)])
        lay = build_layout([(slot, [0] * n, [])], [at], DEV)
        out = torch.empty(n, inner, device=DEV, dtype=ACT[dtype])
        ops.selective_scan(x[at:at + n].to(DEV).contiguous(), low[at:at + n].to(DEV).contiguous(), R,
                           R + N, dt_lin[at:at + n].to(DEV).contiguous(), dt_bias.to(DEV),
                           a_log.to(DEV), d_skip.to(DEV), zz[at:at + n].contiguous(), 5,
                           cache.layer_state(0), lay, N, out)
        outs.append(out.float().cpu())
        at += n
    return torch.cat(outs), cache.layer_state(0)[slot].cpu().view(inner, N)


def _plain_scan(x, low, dt_lin, z, dt_bias, a_log, d_skip, R, N):
    x, low, z = x.double(), low.double(), z.double()
    dt = PN.softplus(dt_lin.double() + dt_bias.double())
    A = -torch.exp(a_log.double())
    S = torch.zeros(x.shape[1], N, dtype=torch.float64)
    y = torch.zeros_like(x)
    for t in range(x.shape[0]):
        B, C = low[t, R:R + N], low[t, R + N:R + 2 * N]
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[None, :]
        y[t] = S @ C + d_skip.double() * x[t]
    return y * PN.silu(z), S


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inner,N,R", [(40, 5, 3), (130, 16, 8), (1, 1, 1), (260, 24, 2), (33, 70, 4), (8, 130, 1)])
def test_selective_scan_whole_in_portions_and_token_by_token(ops, dtype, inner, N, R):
    T = 150
    x, low = _rnd(T, inner, seed=1), _rnd(T, R + 2 * N + 3, seed=2)
    dt_lin, z = _rnd(T, inner, seed=3), _rnd(T, inner, seed=4, s=2.0)
    dt_bias, a_log, d_skip = _rnd(inner, seed=5) - 2.0, _rnd(inner, N, seed=6, s=0.7) - 0.5, _rnd(inner, seed=7) + 1.0
    ref, S = _plain_scan(x, low, dt_lin, z, dt_bias, a_log, d_skip, R, N)
    for pieces in ([T], [2, 61, 1, 2, 64, 3, 17], [1] * T):
        got, state = _scan(ops, dtype, x, low, dt_lin, z, dt_bias, a_log, d_skip, R, N, pieces)
        _close(got, ref, TOL[dtype], f"scan {inner}x{N} in {len(pieces)} pieces")
        _close(state, S, 2e-5, "state after the sequence")


def test_selective_scan_remembers_and_forgets(ops):
    """A channel whose decay is next to nothing still holds its first token after 400; one whose
    decay is strong has lost it."""
    T, inner, N = 400, 2, 3
    x = torch.zeros(T, inner)
    x[0] = 1.0
    low = torch.ones(T, 2 * N)
    dt_lin = torch.zeros(T, inner)
    a_log = torch.tensor([[-20.0] * N, [1.0] * N])         # A = -2e-9 and A = -2.7
    dt_bias, d_skip, z = torch.zeros(inner), torch.zeros(inner), torch.full((T, inner), 30.0)
    ref, _ = _plain_scan(x, low, dt_lin, z, dt_bias, a_log, d_skip, 0, N)
    assert float(ref[-1, 0]) > 0.5 * float(ref[0, 0]) and float(ref[-1, 1]) < 1e-12
    got, _ = _scan(ops, "float32", x, low, dt_lin, z, dt_bias, a_log, d_skip, 0, N, [100] + [1] * 300)
    _close(got, ref, 2e-5, "first token after 400")


# ----------------------------------------------------------------------------- linear attention
def _linear(ops, fused, cols, decay, H, d, dv, pieces):
    T = fused.shape[0]
    cache = _stores("float32", 1, 1, 1, H * d * dv, 64)
    slot, at, outs = cache.alloc_slot(), 0, []
    for n in pieces:
        lay = build_layout([(slot, [0] * n, [])], [at], DEV)
        out = torch.empty(n, H * dv, device=DEV)
        ops.linear_attention(fused[at:at + n].to(DEV).contiguous(), *cols, ACT_SILU, decay.to(DEV),
                             cache.layer_state(0), lay, H, d, dv, out)
        outs.append(out.cpu())
        at += n
    return torch.cat(outs), cache.layer_state(0)[slot].cpu().view(H, d, dv)


def _plain_linear(fused, cols, decay, H, d, dv):
    T = fused.shape[0]
    f = fused.double()
    q = PN.silu(f[:, cols[0]:cols[0] + H * d]).view(T, H, d)
    k = PN.silu(f[:, cols[1]:cols[1] + H * d]).view(T, H, d)
    v = PN.silu(f[:, cols[2]:cols[2] + H * dv]).view(T, H, dv)
    S = torch.zeros(H, d, dv, dtype=torch.float64)
    o = torch.zeros(T, H, dv, dtype=torch.float64)
    for t in range(T):
        S = decay.double()[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o.reshape(T, H * dv), S


@pytest.mark.parametrize("H,d,dv", [(3, 10, 14), (2, 24, 24), (1, 1, 1), (5, 7, 9), (4, 32, 64), (2, 64, 64),
                                    (2, 96, 40), (1, 130, 300), (2, 33, 5)])
def test_linear_attention_whole_in_portions_and_token_by_token(ops, H, d, dv):
    T = 150
    cols = (2, 2 + H * d + 1, 2 + 2 * H * d + 3)
    fused = _rnd(T, cols[2] + H * dv + 4, seed=1)
    decay = torch.linspace(0.5, 1.0, H)
    ref, S = _plain_linear(fused, cols, decay, H, d, dv)
    for pieces in ([T], [2, 61, 1, 2, 64, 3, 17], [1] * T):
        got, state = _linear(ops, fused, cols, decay, H, d, dv, pieces)
        _close(got, ref, 2e-5, f"{H} heads of {d}x{dv} in {len(pieces)} pieces")
        _close(state, S, 2e-5, "state after the sequence")


def test_linear_attention_remembers_by_its_decay(ops):
    """Head 0 (decay 1) returns its first token's value after 400 tokens whose keys are nothing;
    head 1 (decay 0.9) has lost it."""
    T, H, d, dv = 400, 2, 4, 3
    fused = torch.full((T, 2 * H * d + H * dv), -30.0)           # silu(-30) is nothing
    fused[0] = 5.0
    fused[:, :H * d] = 5.0                                        # every query asks
    decay = torch.tensor([1.0, 0.9])
    cols = (0, H * d, 2 * H * d)
    ref, _ = _plain_linear(fused, cols, decay, H, d, dv)
    assert float(ref[-1, 0]) > 0.99 * float(ref[0, 0]) and float(ref[-1, dv]) < 1e-15 * float(ref[0, dv]) + 1e-9
    got, _ = _linear(ops, fused, cols, decay, H, d, dv, [100] + [1] * 300)
    _close(got, ref, 2e-5, "first token after 400")


# ----------------------------------------------------------------------------- batches
def test_a_batch_of_unequal_sequences_is_each_alone(ops):
    """Three sequences on scattered slots, packed with padding rows, through the convolution and
    both recurrences: every sequence's rows are what it gives alone."""
    lens, inner, N, R, H, d, dv, taps = (37, 1, 70), 24, 5, 2, 2, 6, 9, 4
    T = sum(lens)
    n_rows = T + 4
    cache = SequenceCache({}, {0: StateRequest((taps - 1) * inner), 1: StateRequest(inner * N),
                               2: StateRequest(H * d * dv)}, cache_tokens=256, max_seq_len=256,
                          dtype=torch.float32, device=torch.device(DEV), n_slots=6)
    held = [cache.alloc_slot() for _ in range(6)]
    slots = [held[4], held[1], held[3]]
    u, w, b = _rnd(T, inner, seed=1), _rnd(inner, taps, seed=2, s=0.7), _rnd(inner, seed=3)
    low, dt_lin, z = _rnd(T, R + 2 * N, seed=4), _rnd(T, inner, seed=5), _rnd(T, inner, seed=6)
    dt_bias, a_log, d_skip = _rnd(inner, seed=7) - 2, _rnd(inner, N, seed=8) - 0.5, _rnd(inner, seed=9)
    cols = (0, H * d, 2 * H * d)
    fused = _rnd(T, 2 * H * d + H * dv, seed=10)
    decay = torch.tensor([0.8, 0.99])
    pad = lambda t: torch.cat([t, torch.full((n_rows - T, t.shape[1]), float("nan"))]).to(DEV)
    lay = build_layout([(s, [0] * n, []) for s, n in zip(slots, lens)], [0, 0, 0], DEV, pad_rows_to=n_rows)
    assert lay.n_rows == n_rows
    x = torch.empty(n_rows, inner, device=DEV)
    ops.conv_act(pad(u), 0, w.to(DEV), b.to(DEV), taps, ACT_SILU, cache.layer_state(0), lay, x)
    y = torch.empty(n_rows, inner, device=DEV)
    ops.selective_scan(x, pad(low), R, R + N, pad(dt_lin), dt_bias.to(DEV), a_log.to(DEV), d_skip.to(DEV),
                       pad(z), 0, cache.layer_state(1), lay, N, y)
    o = torch.empty(n_rows, H * dv, device=DEV)
    ops.linear_attention(pad(fused), *cols, ACT_SILU, decay.to(DEV), cache.layer_state(2), lay, H, d, dv, o)
    at = 0
    for n in lens:
        sl = slice(at, at + n)
        xs = PN.silu(PN.causal_conv(u[sl].double(), w.double(), b.double()))
        _close(x[sl], xs, 2e-6, "convolution")
        ref, _ = _plain_scan(xs, low[sl], dt_lin[sl], z[sl], dt_bias, a_log, d_skip, R, N)
        _close(y[sl], ref, 2e-5, "scan")
        ref, _ = _plain_linear(fused[sl], cols, decay, H, d, dv)
        _close(o[sl], ref, 2e-5, "linear attention")
        at += n
    # rows of state that belong to no sequence of the step are untouched
    for e in range(3):
        others = [s for s in held if s not in slots]
        assert float(cache.layer_state(e)[others].abs().max()) == 0.0
