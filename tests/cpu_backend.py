"""A stand-in for the kernel library, written with torch CPU ops, for tests of the engine's
HOST logic (batch packing, paging, slots, generation decisions) on a machine without a GPU.
It is a test double only: the package never installs it, and the GPU tests never use it.
Each method has the signature of the same-named method of ``csrc.ops.CudaBackend``.
"""
from __future__ import annotations

import math

import torch


class CpuBackend:
    name = "cpu-test-double"

    def __init__(self):
        self.launches = 0

    def embed_pos(self, tokens, pos, wte, wpe, out, scale=1.0):
        n = out.shape[0]
        tok = tokens[:n].long()
        valid = tok >= 0
        x = wte[tok.clamp(min=0)].float() * scale
        if wpe is not None:
            x = x + wpe[pos[:n].long()].float()
        out.copy_(torch.where(valid[:, None], x, torch.zeros_like(x)))

    def embed_hashed(self, layout, wte, pair, last, out, scale, mul_prev, mul_cur, n_buckets):
        tokens, pos, row_slot = layout.tokens, layout.row_pos, layout.row_slot
        before = last.clone()
        for r in range(out.shape[0]):
            tok, slot, p = int(tokens[r]), int(row_slot[r]), int(pos[r])
            if tok < 0 or slot < 0:
                out[r].zero_()
                continue
            bucket = n_buckets
            if p > 0:
                if r > 0 and int(row_slot[r - 1]) == slot and int(pos[r - 1]) == p - 1:
                    prev = int(tokens[r - 1])
                else:
                    prev = int(before[slot, 0])
                bucket = (prev * mul_prev + tok * mul_cur) % n_buckets
            out[r] = wte[tok].float() * scale + pair[bucket].float()
            more = r + 1 < out.shape[0] and int(row_slot[r + 1]) == slot and int(pos[r + 1]) == p + 1
            if not more:
                last[slot, 0] = float(tok)

    def ln_add(self, y, gamma, eps, residual, next_gamma, next_eps, out_next, out_cast):
        def unit(t, e):
            c = t - t.mean(-1, keepdim=True)
            return c / torch.sqrt((c * c).mean(-1, keepdim=True) + e)
        n = residual.shape[0]
        residual += unit(y[:n], eps) * gamma
        if out_next is not None:
            out_next.copy_((unit(residual, next_eps) * next_gamma).to(out_next.dtype))
        if out_cast is not None:
            out_cast.copy_(residual.to(out_cast.dtype))

    def layernorm(self, x, gamma, beta, eps, out, rows=None):
        n = out.shape[0]
        src = x[:n] if rows is None else x[rows[:n].long().clamp(min=0)]
        mean = src.mean(-1, keepdim=True)
        var = ((src - mean) ** 2).mean(-1, keepdim=True)
        y = (src - mean) / torch.sqrt(var + eps) * gamma
        if beta is not None:
            y = y + beta
        if rows is not None:
            y = torch.where((rows[:n] >= 0)[:, None], y, torch.zeros_like(y))
        out.copy_(y.to(out.dtype))

    def rmsnorm(self, x, gamma, eps, out, rows=None, x_col=0):
        n, d = out.shape
        src = x[:n] if rows is None else x[rows[:n].long().clamp(min=0)]
        src = src[:, x_col:x_col + d]
        y = src / torch.sqrt((src * src).mean(-1, keepdim=True) + eps)
        if gamma is not None:
            y = y * gamma
        if rows is not None:
            y = torch.where((rows[:n] >= 0)[:, None], y, torch.zeros_like(y))
        out.copy_(y.to(out.dtype))

    def rms_add(self, y, gamma, eps, residual, next_gamma, next_eps, out_next, out_cast):
        n = residual.shape[0]
        v = y[:n] / torch.sqrt((y[:n] * y[:n]).mean(-1, keepdim=True) + eps) * gamma
        residual += v
        if out_next is not None:
            x = residual
            out_next.copy_((x / torch.sqrt((x * x).mean(-1, keepdim=True) + next_eps)
                            * next_gamma).to(out_next.dtype))
        if out_cast is not None:
            out_cast.copy_(residual.to(out_cast.dtype))

    def act_rows(self, x, x_col, act, params, out):
        n, d = out.shape
        z = x[:n, x_col:x_col + d].float()
        if act == 5:
            y = torch.tanh(z)
        elif act == 6:
            sp = torch.nn.functional.softplus
            ap, an = sp(params[0]), 0.5 + sp(params[1])
            neg = torch.clamp(z, max=0.0)
            y = torch.where(z > 0, ap * z * z + 0.5 * z, an * (torch.expm1(neg) - neg) + 0.5 * z)
        else:
            y = self._act(z, act)       # what a product's epilogue can apply, or nothing
        out.copy_(y.to(out.dtype))

    def gather_mul(self, g, table, tokens, out):
        n = out.shape[0]
        tok = tokens[:n].long()
        e = table[tok.clamp(min=0)].float()
        y = torch.where((tok >= 0)[:, None], g[:n].float() * e, torch.zeros_like(e))
        out.copy_(y.to(out.dtype))

    @staticmethod
    def _entry(kv, plane, slot, index):
        page = int(kv.block_table[slot, index // kv.page])
        return plane[page, :, index % kv.page, :]

    def qk_norm_rope_append(self, src, q_col, k_col, q_gamma, k_gamma, eps, freq, rot_dims,
                            amplitude, layout, kv, n_heads, q_out, write):
        d, G = kv.head_dim, kv.n_kv_heads
        half = rot_dims // 2

        def turn(x, pos):
            if not rot_dims:
                return x
            ang = (torch.tensor(float(pos), dtype=torch.float32) * freq).float()
            c, s = torch.cos(ang) * amplitude, torch.sin(ang) * amplitude
            u, v = x[:, :half], x[:, half:rot_dims]
            return torch.cat([u * c - v * s, v * c + u * s, x[:, rot_dims:]], dim=-1)

        for r in range(layout.n_rows):
            slot = int(layout.row_slot[r])
            if slot < 0:
                q_out[r].zero_()
                continue
            pos = int(layout.row_pos[r])
            q = src[r, q_col:q_col + n_heads * d].float().view(n_heads, d)
            k = src[r, k_col:k_col + G * d].float().view(G, d)
            qn = q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps) * q_gamma
            kn = k / torch.sqrt((k * k).mean(-1, keepdim=True) + eps) * k_gamma
            q_out[r] = turn(qn, pos).reshape(-1).to(q_out.dtype)
            if write:
                self._entry(kv, kv.k, slot, pos)[:] = turn(kn, pos).to(kv.k.dtype)
                self._entry(kv, kv.v, slot, pos)[:] = k.to(kv.v.dtype)

    def qkv_norm_rope_append(self, src, q_col, k_col, v_col, q_gamma, k_gamma, eps, freq, rot_dims,
                             amplitude, layout, k_store, v_store, n_heads, value_dim, q_out, write):
        d, G = k_store.head_dim, k_store.n_kv_heads
        half = rot_dims // 2

        def turn(x, pos):
            if not rot_dims:
                return x
            ang = (torch.tensor(float(pos), dtype=torch.float32) * freq).float()
            c, s = torch.cos(ang) * amplitude, torch.sin(ang) * amplitude
            u, v = x[:, :half], x[:, half:rot_dims]
            return torch.cat([u * c - v * s, v * c + u * s, x[:, rot_dims:]], dim=-1)

        for r in range(layout.n_rows):
            slot = int(layout.row_slot[r])
            if slot < 0:
                q_out[r].zero_()
                continue
            pos = int(layout.row_pos[r])
            q = src[r, q_col:q_col + n_heads * d].float().view(n_heads, d)
            k = src[r, k_col:k_col + G * d].float().view(G, d)
            if q_gamma is not None:
                q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps) * q_gamma
                k = k / torch.sqrt((k * k).mean(-1, keepdim=True) + eps) * k_gamma
            q_out[r] = turn(q, pos).reshape(-1).to(q_out.dtype)
            if write:
                self._entry(k_store, k_store.k, slot, pos)[:] = turn(k, pos).to(k_store.k.dtype)
                vals = self._values_of(k_store, v_store)
                v = src[r, v_col:v_col + G * value_dim].float().view(G, value_dim)
                self._entry(v_store, vals, slot, pos)[:] = v.to(vals.dtype)

    def attention_masked(self, q, layout, k_store, v_store, n_heads, sink, out, scale, softcap=0.0,
                         window=0, keep_first=0, chunk=0, gate=None, gate_col=0):
        d, dv, G = k_store.head_dim, v_store.head_dim, k_store.n_kv_heads
        group = n_heads // G
        for r in range(layout.n_rows):
            slot = int(layout.row_slot[r])
            if slot < 0:
                out[r].zero_()
                continue
            pos = int(layout.row_pos[r])
            seen = [j for j in range(pos + 1)
                    if (not window or pos - j < window or j < keep_first)
                    and (not chunk or j // chunk == pos // chunk)]
            keys = torch.stack([self._entry(k_store, k_store.k, slot, j).float() for j in seen])
            vals = torch.stack([self._entry(v_store, self._values_of(k_store, v_store), slot, j).float() for j in seen])
            qr = q[r].float().view(n_heads, d)
            for h in range(n_heads):
                s = (keys[:, h // group] @ qr[h]) * scale
                if softcap:
                    s = softcap * torch.tanh(s / softcap)
                m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
                e = torch.exp(s - m)
                den = e.sum() + (torch.exp(sink[h] - m) if sink is not None else 0.0)
                o = (e / den) @ vals[:, h // group]
                if gate is not None:
                    o = o * torch.sigmoid(gate[r, gate_col + h])
                out[r, h * dv:(h + 1) * dv] = o.to(out.dtype)

    def pool_blocks(self, layout, kv, blocks, pool):
        for r in range(layout.n_rows):
            slot = int(layout.row_slot[r])
            pos = int(layout.row_pos[r])
            if slot < 0 or (pos + 1) % pool:
                continue
            ks = torch.stack([self._entry(kv, kv.k, slot, j).float() for j in range(pos + 1 - pool, pos + 1)])
            vs = torch.stack([self._entry(kv, kv.v, slot, j).float() for j in range(pos + 1 - pool, pos + 1)])
            self._entry(blocks, blocks.k, slot, pos // pool)[:] = ks.mean(0).to(blocks.k.dtype)
            self._entry(blocks, blocks.v, slot, pos // pool)[:] = vs.mean(0).to(blocks.v.dtype)

    def attention_pooled(self, q, layout, kv, blocks, n_heads, sink, out, scale, window, pool):
        d, G = kv.head_dim, kv.n_kv_heads
        group = n_heads // G
        for r in range(layout.n_rows):
            slot = int(layout.row_slot[r])
            if slot < 0:
                out[r].zero_()
                continue
            pos = int(layout.row_pos[r])
            lo = max(0, pos + 1 - window) if window > 0 else 0
            keys = [self._entry(kv, kv.k, slot, j).float() for j in range(lo, pos + 1)]
            vals = [self._entry(kv, kv.v, slot, j).float() for j in range(lo, pos + 1)]
            if blocks is not None and window > 0 and pool > 0:
                for b in range(max(0, (pos - window + 1) // pool)):
                    keys.append(self._entry(blocks, blocks.k, slot, b).float())
                    vals.append(self._entry(blocks, blocks.v, slot, b).float())
            keys, vals = torch.stack(keys), torch.stack(vals)          # [n, G, d]
            qr = q[r].float().view(n_heads, d)
            for h in range(n_heads):
                s = (keys[:, h // group] @ qr[h]) * scale
                m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
                e = torch.exp(s - m)
                den = e.sum() + (torch.exp(sink[h] - m) if sink is not None else 0.0)
                out[r, h * d:(h + 1) * d] = ((e / den) @ vals[:, h // group]).to(out.dtype)

    def delta_rule(self, fused, col_r, col_k, col_v, col_g, col_a, decay_logits, a_bias, norm_w,
                   eps, decay_rate, key_eps, layout, state, n_heads, dim, out):
        H, d = n_heads, dim
        hd = H * d
        for r in range(layout.n_rows):        # rows of a sequence come in order of position
            slot = int(layout.row_slot[r])
            if slot < 0:
                out[r].zero_()
                continue
            row = fused[r].float()
            rr = row[col_r:col_r + hd].view(H, d)
            k = row[col_k:col_k + hd].view(H, d)
            v = row[col_v:col_v + hd].view(H, d)
            g = torch.sigmoid(row[col_g:col_g + hd])
            a = torch.sigmoid(row[col_a:col_a + hd] + a_bias).view(H, d)
            w = torch.exp(-decay_rate * torch.sigmoid(decay_logits[r].float())).view(H, d)
            u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + key_eps)
            S = state[slot].view(H, d, d)
            removed = torch.einsum("hk,hkv->hv", u, S)
            S.copy_(w[:, :, None] * S - (a * u)[:, :, None] * removed[:, None, :]
                    + k[:, :, None] * v[:, None, :])
            o = torch.einsum("hkv,hk->hv", S, rr)
            o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps)
            out[r] = (o.reshape(hd) * norm_w * g).to(out.dtype)

    # -- short convolutions, capped attention, linear recurrences (row by row, in order) ---
    @staticmethod
    def _act(x, act):
        if act == 3:
            return x * torch.sigmoid(x)
        if act == 7:
            return torch.relu(x)
        if act == 4:
            return torch.relu(x) ** 2
        if act == 1:
            return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))
        if act == 2:
            return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))
        assert act == 0
        return x

    @staticmethod
    def _conv_row(u, w, taps, state_row, C):
        """One token through the convolution: its result, and the state moved on by one."""
        if taps <= 0:
            return u
        past = state_row.view(taps - 1, C) if taps > 1 else u.new_zeros((0, C))
        window = torch.cat([past, u[None]])                      # [taps, C], oldest first
        y = (window * w.t()).sum(0)
        if taps > 1:
            state_row.copy_(window[1:].reshape(-1))
        return y

    @staticmethod
    def _values_of(k_store, v_store):
        """The plane of values: the second plane when one store holds both."""
        return k_store.v if v_store is k_store else v_store.k

    def conv_rope_append(self, src, col0, w, taps, state, freq, rot_dims, layout, k_store,
                         v_store, n_heads, dv, q_out):
        d, G = k_store.head_dim, k_store.n_kv_heads
        qw, kw = n_heads * d, G * d
        C = qw + kw + G * dv
        taps = int(taps) if w is not None else 0

        def turn(x, pos):
            if not rot_dims:
                return x
            ang = (torch.tensor(float(pos), dtype=torch.float32) * freq).float()
            c, s = torch.cos(ang), torch.sin(ang)
            u, v = x[:, 0:rot_dims:2], x[:, 1:rot_dims:2]
            out = x.clone()
            out[:, 0:rot_dims:2] = u * c - v * s
            out[:, 1:rot_dims:2] = v * c + u * s
            return out

        for r in range(layout.n_rows):
            slot = int(layout.row_slot[r])
            if slot < 0:
                q_out[r].zero_()
                continue
            pos = int(layout.row_pos[r])
            y = self._conv_row(src[r, col0:col0 + C].float(), w, taps,
                               state[slot] if taps > 1 else None, C)
            q_out[r] = turn(y[:qw].view(n_heads, d), pos).reshape(-1).to(q_out.dtype)
            self._entry(k_store, k_store.k, slot, pos)[:] = turn(y[qw:qw + kw].view(G, d), pos).to(k_store.k.dtype)
            self._entry(v_store, self._values_of(k_store, v_store), slot, pos)[:] = y[qw + kw:].view(G, dv).to(v_store.k.dtype)

    def conv_act(self, src, col0, w, bias, taps, act, state, layout, out_f32, out_act=None):
        C = out_f32.shape[1]
        taps = int(taps) if w is not None else 0
        for r in range(layout.n_rows):
            slot = int(layout.row_slot[r])
            if slot < 0:
                out_f32[r].zero_()
                continue
            y = self._conv_row(src[r, col0:col0 + C].float(), w, taps,
                               state[slot] if taps > 1 else None, C)
            if bias is not None:
                y = y + bias
            out_f32[r] = self._act(y, act)
        if out_act is not None and out_act is not out_f32:
            out_act.copy_(out_f32.to(out_act.dtype))

    def attention_capped(self, q, layout, k_store, v_store, n_heads, sink, out, scale, softcap):
        d, dv, G = k_store.head_dim, v_store.head_dim, k_store.n_kv_heads
        group = n_heads // G
        for r in range(layout.n_rows):
            slot = int(layout.row_slot[r])
            if slot < 0:
                out[r].zero_()
                continue
            pos = int(layout.row_pos[r])
            keys = torch.stack([self._entry(k_store, k_store.k, slot, j).float() for j in range(pos + 1)])
            vals = torch.stack([self._entry(v_store, self._values_of(k_store, v_store), slot, j).float() for j in range(pos + 1)])
            qr = q[r].float().view(n_heads, d)
            for h in range(n_heads):
                s = (keys[:, h // group] @ qr[h]) * scale
                if softcap:
                    s = softcap * torch.tanh(s / softcap)
                m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
                e = torch.exp(s - m)
                den = e.sum() + (torch.exp(sink[h] - m) if sink is not None else 0.0)
                out[r, h * dv:(h + 1) * dv] = ((e / den) @ vals[:, h // group]).to(out.dtype)

    def selective_scan(self, x, low, col_b, col_c, dt_lin, dt_bias, a_log, d_skip, z, z_col, state,
                       layout, n_state, out):
        inner, N = x.shape[1], n_state
        A = -torch.exp(a_log.float())
        for r in range(layout.n_rows):
            slot = int(layout.row_slot[r])
            if slot < 0:
                out[r].zero_()
                continue
            dt = torch.nn.functional.softplus(dt_lin[r].float() + dt_bias)
            xr, B, C = x[r].float(), low[r, col_b:col_b + N].float(), low[r, col_c:col_c + N].float()
            S = state[slot].view(inner, N)
            S.copy_(torch.exp(dt[:, None] * A) * S + (dt * xr)[:, None] * B[None, :])
            y = S @ C + d_skip * xr
            zr = z[r, z_col:z_col + inner].float()
            out[r] = (y * zr * torch.sigmoid(zr)).to(out.dtype)

    def linear_attention(self, fused, col_q, col_k, col_v, act, decay, state, layout, n_heads, d, dv,
                         out):
        H = n_heads
        for r in range(layout.n_rows):
            slot = int(layout.row_slot[r])
            if slot < 0:
                out[r].zero_()
                continue
            row = fused[r].float()
            q = self._act(row[col_q:col_q + H * d], act).view(H, d)
            k = self._act(row[col_k:col_k + H * d], act).view(H, d)
            v = self._act(row[col_v:col_v + H * dv], act).view(H, dv)
            S = state[slot].view(H, d, dv)
            S.copy_(decay[:, None, None] * S + k[:, :, None] * v[:, None, :])
            out[r] = torch.einsum("hkv,hk->hv", S, q).reshape(-1)

    def rmsnorm_gated(self, x, gamma, gate, gate_col, eps, out):
        n, d = out.shape
        xr = x[:n].float()
        y = xr / torch.sqrt((xr * xr).mean(-1, keepdim=True) + eps) * gamma
        out.copy_((y * torch.sigmoid(gate[:n, gate_col:gate_col + d].float())).to(out.dtype))

    def rms_pair_add(self, a, gamma_a, b, gamma_b, eps, coef, residual, next_gamma=None,
                     next_eps=0.0, out_next=None):
        def unit(t):
            return t / torch.sqrt((t * t).mean(-1, keepdim=True) + eps)
        residual += coef * (unit(a.float()) * gamma_a + unit(b.float()) * gamma_b)
        if out_next is not None:
            u = residual / torch.sqrt((residual * residual).mean(-1, keepdim=True) + next_eps)
            out_next.copy_((u * next_gamma).to(out_next.dtype))

    @classmethod
    def _gate_up(cls, gate, up, act, param):
        if act == 8:
            g = torch.clamp(gate, max=param)
            return g * torch.sigmoid(1.702 * g) * (torch.clamp(up, -param, param) + 1.0)
        return cls._act(gate, act) * up

    def glu_rows(self, x, gate_col, up_col, act, out, act_param=0.0):
        n, d = out.shape
        out.copy_(self._gate_up(x[:n, gate_col:gate_col + d].float(),
                                x[:n, up_col:up_col + d].float(), act, act_param).to(out.dtype))

    def cast_cols(self, x, out, out_col):
        out[:, out_col:out_col + x.shape[1]] = x.to(out.dtype)

    def latent_append(self, src, col, gamma, eps, layout, kv):
        rank = kv.head_dim
        for r in range(layout.n_rows):
            slot = int(layout.row_slot[r])
            if slot < 0:
                continue
            pos = int(layout.row_pos[r])
            v = src[r, col:col + rank]
            v = v / torch.sqrt((v * v).mean() + eps)
            if gamma is not None:
                v = v * gamma
            page = int(kv.block_table[slot, pos // kv.page])
            kv.k[page, 0, pos % kv.page, :] = v.to(kv.k.dtype)

    def head_linear(self, x, x_col, w, out, layout, gate=None, gate_col=0):
        n = layout.n_rows
        n_heads, n_out, n_in = w.shape
        xs = x[:n, x_col:x_col + n_heads * n_in].float().view(n, n_heads, n_in)
        y = torch.einsum("rhi,hoi->rho", xs, w.float())
        if gate is not None:
            y = y * torch.sigmoid(gate[:n, gate_col:gate_col + n_heads])[:, :, None]
        y = torch.where((layout.row_slot[:n] >= 0)[:, None, None], y, torch.zeros_like(y))
        out[:n].copy_(y.reshape(n, n_heads * n_out).to(out.dtype))

    def attention_latent(self, q, layout, kv, n_heads, sink, out, scale, window=0):
        rank = kv.head_dim
        for r in range(layout.n_rows):
            slot = int(layout.row_slot[r])
            if slot < 0:
                out[r].zero_()
                continue
            pos = int(layout.row_pos[r])
            lo = max(0, pos + 1 - window) if window > 0 else 0
            idx = torch.arange(lo, pos + 1)
            pages = kv.block_table[slot, (idx // kv.page).long()].long()
            c = kv.k[pages, 0, (idx % kv.page).long(), :].float()       # [n, rank]
            a = q[r].float().view(n_heads, rank)
            s = (a @ c.t()) * scale                                      # [heads, n]
            m = s.max(-1).values
            if sink is not None:
                m = torch.maximum(m, sink)
            e = torch.exp(s - m[:, None])
            den = e.sum(-1)
            if sink is not None:
                den = den + torch.exp(sink - m)
            out[r] = ((e / den[:, None]) @ c).reshape(-1).to(out.dtype)

    def moe_route(self, logits, col, n_experts, top, renormalize, layout, idx, weight):
        n = layout.n_rows
        s = torch.softmax(logits[:n, col:col + n_experts].float(), dim=-1)
        order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
        w = torch.gather(s, 1, order)
        if renormalize:
            w = w / w.sum(-1, keepdim=True)
        live = (layout.row_slot[:n] >= 0)[:, None]
        idx.copy_(torch.where(live, order.to(torch.int32), torch.full_like(idx, -1)))
        weight.copy_(torch.where(live, w, torch.zeros_like(w)))

    def moe_route_sigmoid(self, logits, col, bias, n_experts, top, n_groups, keep_groups, group_top,
                          renormalize, norm_eps, out_scale, layout, idx, weight):
        n = layout.n_rows
        s = torch.sigmoid(logits[:n, col:col + n_experts].float())
        c = s + bias if bias is not None else s.clone()
        if n_groups > 1 and keep_groups < n_groups:
            per = n_experts // n_groups
            gs = c.view(n, n_groups, per).topk(min(group_top, per), dim=-1).values.sum(-1)
            kept = torch.sort(gs, dim=-1, descending=True, stable=True).indices[:, :keep_groups]
            ok = torch.zeros((n, n_groups), dtype=torch.bool)
            ok.scatter_(1, kept, True)
            c = c.masked_fill(~ok[:, :, None].expand(n, n_groups, per).reshape(n, n_experts),
                              -math.inf)
        order = torch.sort(c, dim=-1, descending=True, stable=True).indices[:, :top]
        w = torch.gather(s, 1, order)
        if renormalize:
            w = w / (w.sum(-1, keepdim=True) + norm_eps)
        w = w * out_scale
        live = (layout.row_slot[:n] >= 0)[:, None]
        idx.copy_(torch.where(live, order.to(torch.int32), torch.full_like(idx, -1)))
        weight.copy_(torch.where(live, w, torch.zeros_like(w)))

    def moe_group(self, idx, n_experts, offsets, order, place):
        flat = idx.reshape(-1)
        at = 0
        place.fill_(-1)
        for e in range(n_experts):
            offsets[e] = at
            for p in torch.nonzero(flat == e).reshape(-1).tolist():
                order[at] = p
                place[p] = at
                at += 1
        offsets[n_experts] = at

    def moe_linear(self, x, order, row_div, offsets, w, w2, out, act=0, act_param=0.0):
        n_experts = w.shape[0]
        for e in range(n_experts):
            for at in range(int(offsets[e]), int(offsets[e + 1])):
                row = int(order[at]) // row_div if order is not None else at
                v = w[e].float() @ x[row].float()
                if w2 is None and act == 4:
                    v = torch.clamp(v, min=0.0) ** 2
                if w2 is not None and act == 8:
                    v = self._gate_up(v, w2[e].float() @ x[row].float(), act, act_param)
                elif w2 is not None:
                    if act == 3:
                        v = v * torch.sigmoid(v)
                    elif act == 1:
                        v = 0.5 * v * (1 + torch.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3)))
                    elif act == 2:
                        v = 0.5 * v * (1 + torch.erf(v / math.sqrt(2.0)))
                    v = v * (w2[e].float() @ x[row].float())
                out[at] = v.to(out.dtype)

    def moe_combine(self, y, place, weight, residual):
        n, top = weight.shape
        pl = place.reshape(-1)
        for r in range(n):
            for k in range(top):
                at = int(pl[r * top + k])
                if at >= 0:
                    residual[r] += weight[r, k] * y[at]

    def linear(self, x, w, bias, out, act=0, residual=None, norm=None):
        if norm is not None:
            h = torch.empty(x.shape, dtype=norm[3])
            self.layernorm(x, norm[0], norm[1], norm[2], h)
            x = h
        y = x.float() @ w.float().t()
        if bias is not None:
            y = y + bias
        if act == 1:
            y = 0.5 * y * (1 + torch.tanh(0.7978845608028654 * (y + 0.044715 * y ** 3)))
        elif act == 2:
            y = 0.5 * y * (1 + torch.erf(y / math.sqrt(2.0)))
        if residual is not None:
            y = y + residual
        out.copy_(y.to(out.dtype))

    def kv_append(self, src, k_col, v_col, row_slot, row_pos, kv, n_rows):
        w = kv.n_kv_heads * kv.head_dim
        for r in range(n_rows):
            slot = int(row_slot[r])
            if slot < 0:
                continue
            pos = int(row_pos[r])
            page = int(kv.block_table[slot, pos // kv.page])
            kv.k[page, :, pos % kv.page, :] = src[r, k_col:k_col + w].view(kv.n_kv_heads, kv.head_dim)
            kv.v[page, :, pos % kv.page, :] = src[r, v_col:v_col + w].view(kv.n_kv_heads, kv.head_dim)

    def attention_takes(self, q_src, q_col, layout, kv, n_heads, out, scale) -> bool:
        return kv.v is not None

    def attention(self, q_src, q_col, layout, kv, n_heads, out, scale, window=0, append=None,
                  softcap=0.0, sink=None):
        if append:
            self.kv_append(q_src, append[0], append[1], layout.row_slot, layout.row_pos, kv,
                           layout.n_rows)
        hd, group = kv.head_dim, n_heads // kv.n_kv_heads
        for r in range(layout.n_rows):
            slot = int(layout.row_slot[r])
            if slot < 0:
                out[r].zero_()
                continue
            pos = int(layout.row_pos[r])
            lo = max(0, pos + 1 - window) if window > 0 else 0
            idx = torch.arange(lo, pos + 1)
            pages = kv.block_table[slot, (idx // kv.page).long()].long()
            within = (idx % kv.page).long()
            keys = kv.k[pages, :, within, :].float()      # [n, Hk, hd]
            vals = kv.v[pages, :, within, :].float()
            q = q_src[r, q_col:q_col + n_heads * hd].float().view(n_heads, hd)
            for h in range(n_heads):
                s = (keys[:, h // group] @ q[h]) * scale
                if softcap and softcap > 0:
                    s = softcap * torch.tanh(s / softcap)
                if sink is not None:
                    p = torch.softmax(torch.cat([s, sink[h].float().view(1)]), dim=0)[:-1]
                else:
                    p = torch.softmax(s, dim=0)
                out[r, h * hd:(h + 1) * hd] = (p @ vals[:, h // group]).to(out.dtype)

    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).to(torch.int32))

    def sample_temperature(self, logits, temperature, u, out):
        w = logits.double() / max(temperature, 1e-6)
        e = torch.exp(w - w.max(-1, keepdim=True).values)
        c = torch.cumsum(e, -1)
        r = u[:, None] * c[:, -1:]
        idx = (c < r).sum(-1).clamp(max=logits.shape[1] - 1)
        out.copy_(idx.to(torch.int32))

    # The sampling kernels' stand-ins draw with the host's sampler and the number they are given.
    # `hand_back`: mark every row as the top-p kernel marks a row it cannot settle (-2).
    hand_back = False

    def _draw(self, logits, u, out, **kw):
        from nimbus_infer_rs_b200.sampling import SamplingParams
        from nimbus_infer_rs_b200.sampling import host as H
        from nimbus_infer_rs_b200.sampling.device import _Drawn
        p = SamplingParams(**kw)
        for r in range(logits.shape[0]):
            out[r] = int(H.sample(logits[r].numpy(), p, [], _Drawn(float(u[r]))))

    def sample_top_k(self, logits, k, temperature, u, out):
        self._draw(logits, u, out, temperature=temperature, top_k=k)

    def top_p_max_k(self):
        return 1024

    def sample_top_p(self, logits, k, top_p, temperature, u, out):
        if self.hand_back:
            out.fill_(-2)
        else:
            self._draw(logits, u, out, temperature=temperature, top_k=k, top_p=top_p)

    def history_append(self, history, history_len, tokens, row_slot):
        for r in range(tokens.numel()):
            if int(row_slot[r]) >= 0 and int(history_len[r]) < history.shape[1]:
                history[r, int(history_len[r])] = tokens[r]
                history_len[r] += 1

    def repetition_penalty(self, logits, history, history_len, penalty):
        for r in range(logits.shape[0]):
            for tok in set(history[r, :int(history_len[r])].tolist()):
                if 0 <= tok < logits.shape[1]:
                    v = logits[r, tok]
                    logits[r, tok] = v / penalty if v > 0 else v * penalty

    def raise_device_errors(self):
        pass

    def check_device_errors(self):
        pass

    def advance_decode(self, tokens, next_tokens, row_pos, row_slot):
        live = row_slot >= 0
        tokens.copy_(torch.where(live, next_tokens, torch.full_like(tokens, -1)))
        row_pos.add_(live.to(row_pos.dtype))
