"""Pinozen from its equations: a plain, slow restatement in float64, whole sequences at a time,
no cache, no batching, one function per mechanism.  It shares no code with the package: it
reads the raw config.json object and a ``{name: tensor}`` dictionary of the weight file.

Notation: ``T`` tokens, ``D`` width, positions ``0 .. T-1``; a linear weight ``W`` is stored
``[out, in]`` and applied as ``x @ W.T``.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms_unit(x, eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


def softplus(x):
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0)


# ------------------------------------------------------------------------------ short convolution
def causal_conv(u, w, bias=None):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] * u_(t - taps + 1 + j); the last column of
    ``w`` multiplies the current token, and what lies before the first token is zero."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u])
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j]
    return y if bias is None else y + bias


# ------------------------------------------------------------------------------ rotation
def rotary_frequencies(rot):
    """Angular frequency of pair ``i`` of the rotated dimensions.  With ``scaling`` (factor,
    low, high, original): a pair whose wavelength is shorter than ``original / high`` keeps its
    frequency, one longer than ``original / low`` gets ``f / factor``, the ones between a blend
    by ``s = (original / wavelength - low) / (high - low)``."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f
    factor, low, high = float(sc["factor"]), float(sc["low"]), float(sc["high"])
    original = float(sc["original"])
    out = []
    for fi in f.tolist():
        wavelength = 2.0 * math.pi / fi
        if wavelength < original / high:
            out.append(fi)
        elif wavelength > original / low:
            out.append(fi / factor)
        else:
            s = (original / wavelength - low) / (high - low)
            out.append((1.0 - s) * fi / factor + s * fi)
    return torch.tensor(out, dtype=F64)


def rotate_interleaved(x, positions, rot):
    """x [T, heads, dim]: of each head's first ``dims`` numbers, number ``2i`` is paired with
    number ``2i + 1`` and the pair is turned by the angle ``p * f_i``."""
    if not rot:
        return x
    dims = int(rot["dims"])
    f = rotary_frequencies(rot)
    ang = positions.to(F64)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ------------------------------------------------------------------------------ mixers
def capped_sink_attention(q, k, v, scale, softcap, sink):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; position ``i`` sees every ``j <= i``.  A score is
    ``scale * q . k``, then ``softcap * tanh(score / softcap)`` when there is a cap; the
    softmax's denominator also holds ``exp(sink_h)`` (neither scaled nor capped)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for i in range(T):
        for hh in range(H):
            g = hh // (H // G)
            s = (k[:i + 1, g] @ q[i, hh]) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            sk = None if sink is None else sink[hh]
            m = s.max() if sk is None else torch.maximum(s.max(), sk)
            e = torch.exp(s - m)
            den = e.sum() + (torch.exp(sk - m) if sk is not None else 0.0)
            out[i, hh] = (e / den) @ v[:i + 1, g]
    return out


def conv_attention(h, w, mx):
    """The attention branch on normed rows ``h`` [T, D]: projections, a short convolution over
    time on every channel of each, rotation of queries and keys, capped scores, a sink."""
    T = h.shape[0]
    H, G = int(mx["heads"]), int(mx.get("kv_heads", mx["heads"]))
    d, dv = int(mx["dim"]), int(mx.get("vdim", mx["dim"]))
    q, k, v = h @ w["q"].T, h @ w["k"].T, h @ w["v"].T
    if mx.get("conv"):
        q, k, v = causal_conv(q, w["q.conv"]), causal_conv(k, w["k.conv"]), causal_conv(v, w["v.conv"])
    pos = torch.arange(T)
    q = rotate_interleaved(q.view(T, H, d), pos, mx.get("rot"))
    k = rotate_interleaved(k.view(T, G, d), pos, mx.get("rot"))
    o = capped_sink_attention(q, k, v.view(T, G, dv), float(mx["scale"]),
                              float(mx.get("softcap") or 0.0), w.get("sink"))
    return o.reshape(T, H * dv) @ w["o"].T


def selective_scan(h, w, mx):
    """The recurrent branch: ``[x | z] = W_in h``; ``x`` through a short convolution with bias
    and silu; ``[dt | B | C] = W_x x``; ``dt = softplus(W_dt dt + b)`` per channel; ``A =
    -exp(A_log)``; per channel ``c`` and state ``n``: ``S <- exp(dt_c A[c, n]) S + dt_c x_c
    B_n``, ``y_c = sum_n S[c, n] C_n + D_c x_c``; then ``y * silu(z)`` and ``W_o``."""
    T = h.shape[0]
    inner, N, R = int(mx["inner"]), int(mx["state"]), int(mx["dt_rank"])
    xz = h @ w["in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    if mx.get("conv"):
        x = causal_conv(x, w["conv"], w.get("conv.b"))
    x = silu(x)
    low = x @ w["x"].T
    dt = softplus(low[:, :R] @ w["dt"].T + w["dt.b"])           # [T, inner]
    B, C = low[:, R:R + N], low[:, R + N:R + 2 * N]
    A = -torch.exp(w["A_log"])                                   # [inner, N]
    S = torch.zeros(inner, N, dtype=F64)
    y = torch.zeros(T, inner, dtype=F64)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + w["D"] * x[t]
    return (y * silu(z)) @ w["o"].T


def side_by_side(h, w, mx, eps):
    """Two mixers read the same rows; each result is RMS-normed over the width with a weight of
    its own, and the mixer's result is half their sum."""
    wl = {n[len("left."):]: t for n, t in w.items() if n.startswith("left.")}
    wr = {n[len("right."):]: t for n, t in w.items() if n.startswith("right.")}
    a = rms_norm(conv_attention(h, wl, mx["left"]), wl["out"], eps)
    b = rms_norm(selective_scan(h, wr, mx["right"]), wr["out"], eps)
    return 0.5 * (a + b)


def decayed_linear_attention(h, w, mx, eps):
    """``q, k, v = silu(W h)`` per head; ``S_t = decay_h S_(t-1) + k_t v_t^T``, ``o_t = S_t^T
    q_t``; the heads side by side are RMS-normed together, weighted, multiplied by
    ``sigmoid(W_g h)`` and mapped back."""
    T = h.shape[0]
    H, d, dv = int(mx["heads"]), int(mx["dim"]), int(mx.get("vdim", mx["dim"]))
    q = silu(h @ w["q"].T).view(T, H, d)
    k = silu(h @ w["k"].T).view(T, H, d)
    v = silu(h @ w["v"].T).view(T, H, dv)
    decay = torch.tensor([float(x) for x in mx["decay"]], dtype=F64)
    S = torch.zeros(H, d, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = rms_norm(o.reshape(T, H * dv), w["norm"], eps)
    return (o * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


def gated_feed_forward(h, w):
    """``W_down (relu(W_gate h) * (W_up h))``."""
    return (torch.relu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


# ------------------------------------------------------------------------------ the model
def _sub(tensors, prefix):
    return {n[len(prefix):]: t.to(F64) for n, t in tensors.items() if n.startswith(prefix)}


def run_order(cfg):
    """The layers in the order they run: a stretch ``start .. stop-1`` runs ``times`` times in a
    row.  Yields ``(layer, first_of_a_pass)``."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(a)]
    for _ in range(times):
        order += [(i, i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def layer_forward(x, tensors, cfg, i):
    eps = float(cfg["norm"]["eps"])
    l = cfg["layers"][i]
    p = f"l{i}."
    h = rms_norm(x, tensors[p + "norm1"].to(F64), eps)
    w = _sub(tensors, p + "mix.")
    if l["type"] == "parallel":
        x = x + side_by_side(h, w, l["mixer"], eps)
    elif l["type"] == "lightning":
        x = x + decayed_linear_attention(h, w, l["mixer"], eps)
    else:
        raise ValueError(l["type"])
    if l.get("mlp") is not None:
        h = rms_norm(x, tensors[p + "norm2"].to(F64), eps)
        x = x + gated_feed_forward(h, _sub(tensors, p + "mlp."))
    return x


def hidden_states(tokens, tensors, cfg):
    """The stream after every layer run, [runs, T, D], for one sequence from position 0."""
    T = len(tokens)
    tok = torch.as_tensor(tokens, dtype=torch.long)
    x = tensors["embed"].to(F64)[tok] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    if "pos" in tensors:
        x = x + tensors["pos"].to(F64)[:T]
    x0 = x
    out = []
    for i, first in run_order(cfg):
        if first:
            x = torch.cat([x, x0], dim=-1) @ tensors["loop.in"].to(F64).T
        x = layer_forward(x, tensors, cfg, i)
        out.append(x)
    return torch.stack(out)


def logits(tokens, tensors, cfg):
    """Logits at every position of one sequence, [T, vocab]."""
    x = hidden_states(tokens, tensors, cfg)[-1]
    h = rms_norm(x, tensors["final.norm"].to(F64), float(cfg["norm"]["eps"]))
    return (h @ tensors["embed"].to(F64).T) * float(cfg.get("logit_scale", 1.0))
