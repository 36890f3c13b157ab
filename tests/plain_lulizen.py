"""A plain implementation of the Lulizen decoder: whole sequences in float64, no cache, no
batches, one function per mechanism.  It shares no code with the package; the tests compare the
engine with it.

Notation: ``T`` tokens, width ``D``; ``W[name]`` are the tensors of a weight file as float64
(``l<i>.`` prefixes a layer's); a linear map stored ``[out, in]`` acts as ``x @ W.T``.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def as_f64(tensors: dict) -> dict:
    return {k: v.to(F64) for k, v in tensors.items()}


# ----------------------------------------------------------------------------- norms
def layer_norm(x, w, eps):
    """Centre, divide by sqrt(mean squared deviation + eps), scale; no shift."""
    c = x - x.mean(-1, keepdim=True)
    return c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * w


def rms_unit(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


# ----------------------------------------------------------------------------- embedding
def hashed_pair_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the second table for every token: a hash of (token before, token); the extra last
    row for the first token of the sequence."""
    rows = [buckets]
    for before, tok in zip(tokens[:-1], tokens[1:]):
        rows.append((before * mul_prev + tok * mul_cur) % buckets)
    return rows


def embed(tokens, W, cfg):
    x = W["embed"][torch.tensor(tokens)]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        x = x + W["bigram"][torch.tensor(hashed_pair_rows(list(tokens), bg["buckets"],
                                                          bg["mul_prev"], bg["mul_cur"]))]
    return x


# ----------------------------------------------------------------------------- attention
def rotate_halves(x, dims, base):
    """x: [T, heads, d].  Of each head's first ``dims`` numbers, number i and number i + dims/2
    are one pair, turned by the angle t * base^(-2i/dims) at position t."""
    if not dims:
        return x
    half = dims // 2
    T = x.shape[0]
    rate = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = torch.arange(T, dtype=F64)[:, None] * rate[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def visible(T, kind, mask):
    """Boolean [T, T]: row i, column j is True where position i sees position j."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if not mask:
        return ok
    size = mask["size"]
    if kind == "attention":
        return ok & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))
    return ok & ((i - j < size) | (j < mask.get("keep_first", 0)))


def attend(q, k, v, see, scale, cap, sink):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; ``see`` [T, T]; returns [T, H, dv].  ``sink``:
    one logit per head that only enlarges the softmax's denominator, or None."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~see, -math.inf)
        top = s.max(-1, keepdim=True).values
        if sink is not None:
            top = torch.maximum(top, sink[h])
        e = torch.exp(s - top)
        total = e.sum(-1, keepdim=True)
        if sink is not None:
            total = total + torch.exp(sink[h] - top)
        out[:, h] = (e / total) @ v[:, g]
    return out


def attention_mixer(x, W, p, kind, m, eps):
    """Both kinds of mixer: ``attention`` norms q and k per head, masks by blocks and has a sink;
    ``attention_2`` masks by a window that keeps first tokens and gates each head's result."""
    T = x.shape[0]
    H, G = m["heads"], m.get("kv_heads", m["heads"])
    d, dv = m["dim"], m.get("vdim", m["dim"])
    q = (x @ W[p + "q"].T).view(T, H, d)
    k = (x @ W[p + "k"].T).view(T, G, d)
    v = (x @ W[p + "v"].T).view(T, G, dv)
    if kind == "attention":
        q, k = rms_unit(q, W[p + "q.norm"], eps), rms_unit(k, W[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot:
        q, k = rotate_halves(q, rot["dims"], rot["base"]), rotate_halves(k, rot["dims"], rot["base"])
    o = attend(q, k, v, visible(T, kind, m.get("mask")), m.get("scale", d ** -0.5),
               m.get("softcap"), W[p + "sink"] if kind == "attention" else None)
    if kind == "attention_2":
        o = o * torch.sigmoid(x @ W[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ W[p + "o"].T


# ----------------------------------------------------------------------------- feed-forward
def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def dense_feed_forward(x, W, p):
    return (gelu_tanh(x @ W[p + "gate"].T) * (x @ W[p + "up"].T)) @ W[p + "down"].T


def expert(x, W, p, limit):
    """A small gated feed-forward whose halves are bounded before they meet."""
    g = x @ W[p + "gate"].T
    u = x @ W[p + "up"].T
    if limit is not None:
        g, u = torch.clamp(g, max=limit), torch.clamp(u, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def choose_experts(z, bias, top, groups, scale, follow=None, margin=0.0):
    """z: router logits [T, E].  Returns (indices [T, top], weights [T, top]).  Choice by
    sigmoid(z) + bias among the experts of the best groups, weights from sigmoid(z) alone.

    ``follow`` [T, top]: what another implementation chose.  A row whose choice is a close call
    (the last kept and the first left-out group, or the last chosen and the first left-out
    expert, are within ``margin`` of each other) takes that choice instead of its own: rounding
    may settle a close call either way."""
    T, E = z.shape
    s = torch.sigmoid(z)
    c = s + bias if bias is not None else s.clone()
    close = torch.zeros(T, dtype=torch.bool)
    if groups:
        n, keep = groups["count"], groups["keep"]
        per = E // n
        by_group = c.view(T, n, per)
        score = by_group.sort(-1, descending=True).values[:, :, :2].sum(-1)
        ranked = torch.sort(score, dim=-1, descending=True, stable=True)
        if keep < n:
            close |= (ranked.values[:, keep - 1] - ranked.values[:, keep]) < margin
        ok = torch.zeros(T, n, dtype=torch.bool)
        ok.scatter_(1, ranked.indices[:, :keep], True)
        c = c.masked_fill(~ok.repeat_interleave(per, dim=1), -math.inf)
    ranked = torch.sort(c, dim=-1, descending=True, stable=True)
    if top < E:
        close |= (ranked.values[:, top - 1] - ranked.values[:, top]) < margin
    idx = ranked.indices[:, :top]
    if follow is not None:
        idx = torch.where(close[:, None], follow.to(idx.dtype), idx)
    w = s.gather(1, idx)
    return idx, w / (w.sum(-1, keepdim=True) + 1e-20) * scale


def routed_feed_forward(x, W, p, f, follow=None, margin=0.0):
    r = f["router"]
    bias = W.get(p + "correction")
    # the router reads the rows as the engine's product sees them in a 32-bit run: unrounded
    idx, w = choose_experts(x @ W[p + "router"].T, bias, r["top"], r.get("groups"), r.get("scale", 1.0),
                            follow, margin)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for e, a in zip(idx[t].tolist(), w[t]):
            out[t] += a * expert(x[t:t + 1], W, f"{p}e{e}.", f["expert"].get("limit"))[0]
    if f.get("shared"):
        out = out + expert(x, W, p + "shared.", f["shared"].get("limit"))
    return out


# ----------------------------------------------------------------------------- the model
def owner(cfg, i):
    while cfg["layers"][i].get("weights_of") is not None:
        i = cfg["layers"][i]["weights_of"]
    return i


def layer_forward(x, W, cfg, i, follow=None, margin=0.0):
    L, eps = cfg["layers"][i], cfg["norm"]["eps"]
    p = f"l{owner(cfg, i)}."
    y = attention_mixer(layer_norm(x, W[p + "norm1"], eps), W, p + "mix.", L["type"], L["mixer"], eps)
    x = x + layer_norm(y, W[p + "norm1b"], eps)
    f = L.get("mlp")
    if f:
        h = layer_norm(x, W[p + "norm2"], eps)
        y = dense_feed_forward(h, W, p + "mlp.") if f["kind"] == "dense" \
            else routed_feed_forward(h, W, p + "mlp.", f, follow, margin)
        x = x + layer_norm(y, W[p + "norm2b"], eps)
    return x


def hidden_states(tokens, W, cfg, routed=None, margin=0.0):
    """The stream after every layer run, [runs, T, D].  ``routed``: for every layer run with
    routed experts, in order, the experts another implementation chose ([T, top]); close calls
    follow it (:func:`choose_experts`)."""
    W = as_f64(W)
    x = embed(tokens, W, cfg)
    out = []
    calls = iter(routed) if routed is not None else None
    for i, L in enumerate(cfg["layers"]):
        follow = None
        if calls is not None and L.get("mlp") and L["mlp"]["kind"] == "moe":
            follow = next(calls)[:len(tokens)]
        x = layer_forward(x, W, cfg, i, follow, margin)
        out.append(x)
    return torch.stack(out)


def logits(tokens, W, cfg, routed=None, margin=0.0):
    W = as_f64(W)
    x = hidden_states(tokens, W, cfg, routed, margin)[-1]
    return layer_norm(x, W["final.norm"], cfg["norm"]["eps"]) @ W["head"].T
