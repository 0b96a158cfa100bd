"""A stand-in for the kernel library with the same methods, computed with torch on the CPU.

It exists so that the host-side logic (step tables, cache manager, scheduler, engine) can be exercised by the
tests that run without a GPU. It is test code only: the package has no CPU path and never imports this.
"""
from __future__ import annotations

import math

import torch

from tests.plain import qwen3_plain as plain


class FakeKernels:
    launches = 0
    library_launches = 0

    def embedding(self, table, ids):
        return table[ids.long()].clone()

    def rms_norm(self, x, w, eps, rows=None):
        if rows is not None:
            x = x[rows.long()]
        xf = x.float()
        y = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * w.float()
        return y.to(x.dtype)

    def add_rms_norm(self, x, residual, w, eps, rows=None):
        s = (x.float() + residual.float()).to(x.dtype)
        if rows is None:
            residual.copy_(s)
        return self.rms_norm(s, w, eps, rows)

    def silu_mul(self, x, block=0):
        i = x.shape[1] // 2
        if block:
            x = x.reshape(x.shape[0], i // block, 2, block).permute(0, 2, 1, 3).reshape(x.shape[0], 2 * i)
        g, u = x[:, :i].float(), x[:, i:].float()
        return (g / (1 + torch.exp(-g)) * u).to(x.dtype)

    def qk_norm_rope_cache(self, qkv, q_heads, kv_heads, head_dim, *, q_w, k_w, eps, inv_freq, rotary_dim, positions,
                           k_pool=None, v_pool=None, slot_mapping=None, page_size=0, write_kv=True, cos_sin=None):
        T = qkv.shape[0]
        d = head_dim
        q = qkv[:, : q_heads * d].reshape(T, q_heads, d).float()

        def norm(x, w):
            return x if w is None else x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.float()

        def rope(x):
            if not rotary_dim:
                return x
            half = rotary_dim // 2
            if cos_sin is not None:     # the step's own table of cosines and sines [T, half, 2]
                c, s = cos_sin[:, None, :, 0].float(), cos_sin[:, None, :, 1].float()
            else:
                ang = positions.double()[:, None] * inv_freq[None, :]
                c, s = torch.cos(ang)[:, None, :].float(), torch.sin(ang)[:, None, :].float()
            x1, x2 = x[..., :half], x[..., half:rotary_dim]
            out = x.clone()
            out[..., :half] = x1 * c - x2 * s
            out[..., half:rotary_dim] = x2 * c + x1 * s
            return out

        q = rope(norm(q, q_w)).to(qkv.dtype)
        if write_kv:
            k = qkv[:, q_heads * d : (q_heads + kv_heads) * d].reshape(T, kv_heads, d).float()
            v = qkv[:, (q_heads + kv_heads) * d :].reshape(T, kv_heads, d)
            k = rope(norm(k, k_w)).to(qkv.dtype)
            for t in range(T):
                slot = int(slot_mapping[t])
                if slot < 0:
                    continue
                page, off = divmod(slot, page_size)
                k_pool[page, :, off, :] = k[t]
                v_pool[page, :, off, :] = v[t]
        return q.contiguous()

    def paged_attention_generic(self, q, k_pool, v_pool, positions, token_row, kv_indptr, kv_indices, scale, window):
        T, nq, d = q.shape
        nkv, page = k_pool.shape[1], k_pool.shape[2]
        group = nq // nkv
        out = torch.zeros(T, nq * d, dtype=q.dtype)
        for t in range(T):
            pos = int(positions[t])
            b = int(token_row[t])
            pages = kv_indices[int(kv_indptr[b]) : int(kv_indptr[b + 1])]
            lo = max(0, pos - window + 1) if window else 0
            js = list(range(lo, pos + 1))
            kk = torch.stack([k_pool[int(pages[j // page]), :, j % page, :] for j in js]).float()  # [n, nkv, d]
            vv = torch.stack([v_pool[int(pages[j // page]), :, j % page, :] for j in js]).float()
            for h in range(nq):
                s = (kk[:, h // group, :] @ q[t, h].float()) * scale
                p = torch.softmax(s, 0)
                out[t, h * d : (h + 1) * d] = (p @ vv[:, h // group, :]).to(q.dtype)
        return out

    # ---- the wide stream's ends and norm
    def embedding_scaled(self, table, ids, scale):
        return table[ids.long()].float() * scale

    def layer_norm(self, stream, w, b, eps, out_dtype, addend=None, rows=None):
        s = stream if addend is None else stream + addend.float()
        if addend is not None and rows is None:
            stream.copy_(s)
        if rows is not None:
            s = s[rows.long()]
        mu = s.mean(-1, keepdim=True)
        d = s - mu
        return (d * torch.rsqrt((d * d).mean(-1, keepdim=True) + eps) * w + b).to(out_dtype)

    def softcap_(self, logits, cap):
        return logits.copy_(cap * torch.tanh(logits / cap))

    def gemm_simt_batched(self, a, w, out):
        out.copy_(torch.bmm(a.float(), w.float().transpose(1, 2)).to(out.dtype))
        return out

    # ---- latent attention
    def latent_prepare(self, q, down, pool, latent_w, inv_freq, rotary_dim, positions, slot_mapping, heads, nope, rope, rank, eps, page_size):
        T = q.shape[0]
        half = rotary_dim // 2
        if inv_freq is None:      # no rotated part
            inv_freq = torch.zeros(0, dtype=torch.float64)
        ang = positions.double()[:, None] * inv_freq[None, :]
        c, s = torch.cos(ang).float(), torch.sin(ang).float()

        def turn(v):        # [..., rope] float32, rotated in its first rotary_dim elements
            u, w2 = v[..., :half].clone(), v[..., half:rotary_dim].clone()
            shape = [T] + [1] * (v.dim() - 2) + [half]
            v[..., :half] = u * c.reshape(shape) - w2 * s.reshape(shape)
            v[..., half:rotary_dim] = w2 * c.reshape(shape) + u * s.reshape(shape)
            return v

        qv = q.view(T, heads, nope + rope)
        qv[:, :, nope:] = turn(qv[:, :, nope:].float()).to(q.dtype)
        if down is not None:
            lat = down[:, :rank].float()
            lat = lat * torch.rsqrt((lat * lat).mean(-1, keepdim=True) + eps) * latent_w
            entry = torch.cat([lat, turn(down[:, rank:].float())], -1).to(pool.dtype)
            for t in range(T):
                slot = int(slot_mapping[t])
                if slot >= 0:
                    pool[slot // page_size, 0, slot % page_size] = entry[t]

    def latent_attention(self, q_latent, q, pool, positions, token_row, kv_indptr, kv_indices, heads, nope, rope, rank, scale, window, kv_cap=0, few_rows=False, q_indptr=None):
        T = q.shape[0]
        page = pool.shape[2]
        out = torch.zeros(heads, T, rank, dtype=q.dtype)
        qr = q.view(T, heads, nope + rope)[:, :, nope:].float()
        for t in range(T):
            pos, b = int(positions[t]), int(token_row[t])
            if pos < 0:
                continue
            pages = kv_indices[int(kv_indptr[b]) : int(kv_indptr[b + 1])]
            lo = max(0, pos - window + 1) if window else 0
            e = torch.stack([pool[int(pages[j // page]), 0, j % page] for j in range(lo, pos + 1)]).float()    # [n, rank + rope]
            sc = (q_latent[:, t].float() @ e[:, :rank].T + qr[t] @ e[:, rank:].T) * scale                    # [heads, n]
            out[:, t] = (torch.softmax(sc, -1) @ e[:, :rank]).to(q.dtype)
        return out

    # ---- mamba-2
    def mamba2_conv(self, u, col, channels, w, b, state, conv_off, token_row, q_indptr, slots, activation="silu"):
        T, taps = u.shape[0], w.shape[1]
        out = torch.zeros(T, channels, dtype=torch.float32)
        for t in range(T):
            r = int(token_row[t])
            start, slot = int(q_indptr[r]), int(slots[r])
            acc = b.clone()
            for k in range(taps):
                i = t - (taps - 1) + k
                if i >= start:
                    v = u[i, col : col + channels].float()
                else:
                    j = i - start + (taps - 1)
                    v = state[slot, conv_off + j * channels : conv_off + (j + 1) * channels]
                acc = acc + w[:, k] * v
            out[t] = acc / (1 + torch.exp(-acc)) if activation == "silu" else acc
        return out.to(u.dtype)

    def mamba2_conv_state(self, u, col, channels, taps, state, conv_off, q_indptr, slots):
        keep = taps - 1
        for r in range(slots.numel()):
            start, end, slot = int(q_indptr[r]), int(q_indptr[r + 1]), int(slots[r])
            if end == start:
                continue
            old = state[slot, conv_off : conv_off + keep * channels].reshape(keep, channels)
            both = torch.cat([old, u[start:end, col : col + channels].float()])
            state[slot, conv_off : conv_off + keep * channels] = both[both.shape[0] - keep :].reshape(-1)

    def mamba2_scan(self, xbc, u, dt_col, dt_bias, a_log, d, state, q_indptr, slots, heads, P, N, groups):
        T = xbc.shape[0]
        inner, per = heads * P, heads // groups
        y = torch.zeros(T, inner, dtype=torch.float32)
        for r in range(slots.numel()):
            slot = int(slots[r])
            S = state[slot, : heads * N * P].reshape(heads, N, P).clone()
            for t in range(int(q_indptr[r]), int(q_indptr[r + 1])):
                dt = torch.nn.functional.softplus(u[t, dt_col : dt_col + heads].float() + dt_bias, threshold=30.0)
                decay = torch.exp(-torch.exp(a_log) * dt)
                x = xbc[t, :inner].float().reshape(heads, P)
                B = xbc[t, inner : inner + groups * N].float().reshape(groups, N).repeat_interleave(per, 0)
                C = xbc[t, inner + groups * N :].float().reshape(groups, N).repeat_interleave(per, 0)
                S = decay[:, None, None] * S + dt[:, None, None] * B[:, :, None] * x[:, None, :]
                y[t] = ((S * C[:, :, None]).sum(1) + d[:, None] * x).reshape(-1)
            state[slot, : heads * N * P] = S.reshape(-1)
        return y

    def gated_group_norm(self, y, u, w, groups, eps, out_dtype):
        T, inner = y.shape
        z = u[:, :inner].float()
        g = (y * (z / (1 + torch.exp(-z)))).reshape(T, groups, inner // groups)
        g = g * torch.rsqrt((g * g).mean(-1, keepdim=True) + eps)
        return (g.reshape(T, inner) * w).to(out_dtype)

    # ---- routed experts
    def moe_router_logits(self, x, w):
        return x.float() @ w.float().t()

    def moe_route(self, logits, top, score="sigmoid", correction=None, scale=1.0, routed=None, real=None):
        from types import SimpleNamespace
        T, C = logits.shape
        E = C if routed is None else routed
        if score == "sigmoid":
            s = torch.sigmoid(logits)
            choice = logits                          # by logit: the sigmoid saturates in 32-bit
        else:
            s = torch.softmax(logits[:, :E].float(), dim=-1)
            choice = s + (correction.float() if correction is not None else 0.0)
            s = s * scale
        pairs = []
        for t in range(T):
            for e in sorted(range(E), key=lambda e: (-float(choice[t, e]), e))[:top]:
                pairs.append((e, t, float(s[t, e])))
        order = sorted(range(len(pairs)), key=lambda i: (pairs[i][0], i))
        inverse = torch.zeros(len(pairs), dtype=torch.int32)
        for dest, i in enumerate(order):
            inverse[i] = dest
        return SimpleNamespace(top=top, token=torch.tensor([pairs[i][1] for i in order], dtype=torch.int32),
                               weight=torch.tensor([pairs[i][2] for i in order], dtype=torch.float32),
                               expert=[pairs[i][0] for i in order], inverse=inverse, real=E if real is None else real)

    def moe_gather_scale(self, x, route, scale=True):
        rows = x[route.token.long()]
        return (rows.float() * route.weight[:, None]).to(x.dtype) if scale else rows.clone()

    @staticmethod
    def _gate_fn(g, u, activation, limit):
        if activation == "silu":
            return g / (1 + torch.exp(-g)) * u
        if activation == "gelu_tanh":
            return 0.5 * g * (1 + torch.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3))) * u
        g, u = torch.clamp(g, max=limit), torch.clamp(u, min=-limit, max=limit)
        return g * torch.sigmoid(1.702 * g) * (u + 1)

    def gated_act_mul(self, x, activation, limit=0.0, block=0):
        i = x.shape[1] // 2
        return self._gate_fn(x[:, :i].float(), x[:, i:].float(), activation, limit).to(x.dtype)

    def moe_expert_gate_up(self, xs, gate, up, route, gate_up=None, activation="silu", limit=0.0):
        out = torch.zeros(xs.shape[0], gate.shape[1], dtype=xs.dtype)
        for i, e in enumerate(route.expert):
            if e >= getattr(route, "real", 1 << 30):
                continue                              # an identity expert has no weights
            g, u2 = gate[e].float() @ xs[i].float(), up[e].float() @ xs[i].float()
            out[i] = self._gate_fn(g, u2, activation, limit).to(xs.dtype)
        return out

    def moe_expert_down(self, act, down, route):
        out = torch.zeros(act.shape[0], down.shape[1], dtype=act.dtype)
        for i, e in enumerate(route.expert):
            if e < getattr(route, "real", 1 << 30):
                out[i] = (down[e].float() @ act[i].float()).to(act.dtype)
        return out

    def moe_combine_weighted(self, ys, route, x, shared=None, gate_logits=None):
        T = x.shape[0]
        rows = ys.float()
        for i, e in enumerate(route.expert):
            if e >= route.real:
                rows[i] = x[int(route.token[i])].float()
        out = (rows * route.weight[:, None])[route.inverse.long()].reshape(T, route.top, -1).sum(1)
        if shared is not None:
            g = torch.sigmoid(gate_logits[:, -1:].float()) if gate_logits is not None else 1.0
            out = out + g * shared.float()
        return out.to(ys.dtype)

    # ---- residual streams
    def stream_step(self, streams, norm_w, eps, out_dtype, read=None, y=None, mix=None, write=None, init_from=None, rows=None):
        if init_from is not None:
            streams.copy_(init_from.float()[:, None, :].expand_as(streams))
        x = streams
        if y is not None:
            x = torch.einsum("sr,tsw->trw", mix.float(), streams) + write.float()[None, :, None] * y.float()[:, None, :]
            if rows is None:
                streams.copy_(x)
        if rows is not None:
            x = x[rows.long()]
        u = x.sum(1) if read is None else torch.einsum("s,tsw->tw", read.float(), x)
        return (u * torch.rsqrt((u * u).mean(-1, keepdim=True) + eps) * norm_w.float()).to(out_dtype)

    # ---- attention with a sink
    def sink_attention_prepare(self, qkv, k_pool, v_pool, inv_freq, rotary_dim, positions, slot_mapping, heads, kv_heads, dim, vdim, eps, page_size,
                               halves=False):
        T = qkv.shape[0]
        Q, K = heads * dim, kv_heads * dim

        def turn(x):           # [T, n, dim] float32
            if rotary_dim:
                ang = positions.double()[:, None] * inv_freq[None, :]
                c, s = torch.cos(ang)[:, None, :].float(), torch.sin(ang)[:, None, :].float()
                first, second = (slice(0, rotary_dim // 2), slice(rotary_dim // 2, rotary_dim)) if halves else (slice(0, rotary_dim, 2), slice(1, rotary_dim, 2))
                u, v = x[..., first].clone(), x[..., second].clone()
                x[..., first] = u * c - v * s
                x[..., second] = v * c + u * s
            if eps is not None:
                x = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
            return x

        qkv[:, :Q] = turn(qkv[:, :Q].float().reshape(T, heads, dim)).reshape(T, Q).to(qkv.dtype)
        k = turn(qkv[:, Q : Q + K].float().reshape(T, kv_heads, dim)).to(qkv.dtype)
        v = qkv[:, Q + K :].reshape(T, kv_heads, vdim)
        for t in range(T):
            slot = int(slot_mapping[t])
            if slot < 0:
                continue
            page, off = divmod(slot, page_size)
            if v_pool is None:
                k_pool[page, :, off, :dim] = k[t]
                k_pool[page, :, off, dim:] = v[t]
            else:
                k_pool[page, :, off, :] = k[t]
                v_pool[page, :, off, :] = v[t]

    def sink_attention(self, qkv, k_pool, v_pool, positions, token_row, kv_indptr, kv_indices, heads, kv_heads, dim, vdim, scale, sink, kv_cap=0,
                       window=None, softcap=0.0):
        T = qkv.shape[0]
        page_size = k_pool.shape[2]
        out = torch.zeros(T, heads * vdim, dtype=qkv.dtype)
        group = heads // kv_heads
        for t in range(T):
            pos = int(positions[t])
            if pos < 0:
                continue
            r = int(token_row[t])
            pages = kv_indices[int(kv_indptr[r]) : int(kv_indptr[r + 1])].long()
            lo = max(0, pos - window + 1) if window else 0
            first_page = lo // page_size            # pages before it may have been given back (entry -1): never touched
            pages, lo = pages[first_page:], lo - first_page * page_size
            hi = pos + 1 - first_page * page_size
            entries = k_pool[pages].permute(1, 0, 2, 3).reshape(kv_heads, -1, k_pool.shape[3])[:, lo:hi].float()
            keys = entries[..., :dim]
            vals = (entries[..., dim:] if v_pool is None
                    else v_pool[pages].permute(1, 0, 2, 3).reshape(kv_heads, -1, vdim)[:, lo:hi].float())
            assert (pages[lo // page_size :] >= 0).all(), "a page inside the window was given back"
            q = qkv[t, : heads * dim].float().reshape(heads, dim)
            for h in range(heads):
                s = (keys[h // group] @ q[h]) * scale
                if softcap:
                    s = softcap * torch.tanh(s / softcap)
                m = torch.clamp(s.max(), min=0.0) if sink else s.max()
                e = torch.exp(s - m)
                out[t, h * vdim : (h + 1) * vdim] = ((e / (e.sum() + (torch.exp(-m) if sink else 0.0))) @ vals[h // group]).to(qkv.dtype)
        return out

    # ---- a 32-bit stream with root-mean-square norms, a hashed pair embedding, token inputs
    def pair_embedding(self, table, pairs, ids, positions, token_row, q_indptr, slots, state, buckets, mul_prev, mul_cur):
        T = ids.numel()
        out = torch.zeros(T, table.shape[1], dtype=torch.float32)
        for t in range(T):
            r = int(token_row[t])
            if int(positions[t]) <= 0:
                row = buckets
            else:
                prev = int(ids[t - 1]) if t > int(q_indptr[r]) else int(state[int(slots[r]), 0])
                row = (prev * mul_prev + int(ids[t]) * mul_cur) % buckets
            out[t] = table[int(ids[t])].float() + pairs[row].float()
        return out

    def last_token_store(self, ids, q_indptr, slots, state):
        for r in range(slots.numel()):
            lo, hi = int(q_indptr[r]), int(q_indptr[r + 1])
            if hi > lo:
                state[int(slots[r]), 0] = int(ids[hi - 1])

    def wide_rms_norm(self, stream, w, eps, out_dtype, addend=None, extra=None, rows=None):
        s = stream
        if addend is not None:
            s = s + addend.float()
        if extra is not None:
            s = s + extra
        if rows is None and s is not stream:
            stream.copy_(s)
        if rows is not None:
            s = s[rows.long()]
        if w is not None:
            s = s * torch.rsqrt((s * s).mean(-1, keepdim=True) + eps) * w.float()
        return s.to(out_dtype)

    def normed_mean(self, xs, ws, eps):
        acc = 0
        for x, w in zip(xs, ws):
            xf = x.float()
            acc = acc + xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * w.float()
        return (acc / len(xs)).to(xs[0].dtype)

    def add_bias_(self, y, bias):
        y += bias.to(y.dtype)
        return y

    def gelu_mul_rows(self, gate, table, ids):
        g = gate.float()
        act = 0.5 * g * (1 + torch.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3)))
        return (act * table[ids.long()].float()).to(gate.dtype)

    # ---- the gated linear recurrence
    def gated_recurrence_scan(self, u, gates, yx, gate_bias, decay, state, q_indptr, slots, width, blocks):
        T, bw = u.shape[0], width // blocks
        out = torch.zeros(T, width, dtype=u.dtype)
        arg = gates.float() + gate_bias[:, None, :]                      # [blocks, T, 2 bw]
        r = torch.sigmoid(arg[:, :, :bw]).permute(1, 0, 2).reshape(T, width)
        i = torch.sigmoid(arg[:, :, bw:]).permute(1, 0, 2).reshape(T, width)
        a = torch.exp(-decay * r)
        drive = torch.sqrt(-torch.expm1(-2.0 * decay * r)) * i * u.float()        # 1 - a^2 without cancellation where a is near one
        y = yx[:, :width].float()
        y = 0.5 * y * (1 + torch.tanh(math.sqrt(2 / math.pi) * (y + 0.044715 * y ** 3)))
        for row in range(slots.numel()):
            lo, hi = int(q_indptr[row]), int(q_indptr[row + 1])
            S = state[int(slots[row]), :width]
            for t in range(lo, hi):
                S.copy_(a[t] * S + drive[t])
                out[t] = (S * y[t]).to(u.dtype)
        return out

    # ---- the matrix memory
    def matrix_memory_scan(self, qkvg, gates, state, q_indptr, slots, heads, dim, vdim, cap, floor):
        T = qkvg.shape[0]
        QK = heads * dim
        q = qkvg[:, :QK].float().reshape(T, heads, dim) * dim ** -0.5
        k = qkvg[:, QK : 2 * QK].float().reshape(T, heads, dim)
        v = qkvg[:, 2 * QK : 2 * QK + heads * vdim].float().reshape(T, heads, vdim)
        gi = cap * torch.tanh(gates[:, :heads] / cap)
        gf = torch.nn.functional.logsigmoid(cap * torch.tanh(gates[:, heads:] / cap))
        out = torch.zeros(T, heads * vdim, dtype=torch.float32)
        per = dim * vdim + dim + 1
        for row in range(slots.numel()):
            lo, hi = int(q_indptr[row]), int(q_indptr[row + 1])
            st = state[int(slots[row])].view(heads, per)
            for t in range(lo, hi):
                S, n, m = st[:, : dim * vdim].reshape(heads, dim, vdim), st[:, dim * vdim : dim * vdim + dim], st[:, -1]
                new = torch.maximum(gf[t] + m, gi[t])
                keep, take = torch.exp(gf[t] + m - new), torch.exp(gi[t] - new)
                S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
                n = keep[:, None] * n + take[:, None] * k[t]
                num = torch.einsum("hdv,hd->hv", S, q[t])
                den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-new)) + floor
                out[t] = (num / den[:, None]).reshape(-1)
                st.copy_(torch.cat([S.reshape(heads, -1), n, new[:, None]], dim=1))
        return out

    def head_norm_gate(self, o, u, col, w, heads, eps, out_dtype, gate="sigmoid"):
        T, V = o.shape
        x = o.reshape(T, heads, V // heads)
        x = (x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)).reshape(T, V)
        if w is not None:
            x = x * w.float()
        g = u[:, col : col + V].float()
        return (x * torch.sigmoid(g) * (g if gate == "silu" else 1.0)).to(out_dtype)

    # ---- retention
    def retention_prepare(self, u, inv_freq, rotary_dim, positions, heads, dim, k_scale):
        T = u.shape[0]
        x = u[:, : 2 * heads * dim].float().reshape(T, 2 * heads, dim).clone()
        if rotary_dim:
            half = rotary_dim // 2
            ang = positions.double()[:, None] * inv_freq[None, :]
            c, s = torch.cos(ang)[:, None, :].float(), torch.sin(ang)[:, None, :].float()
            a, b = x[..., :half].clone(), x[..., half:rotary_dim].clone()
            x[..., :half] = a * c - b * s
            x[..., half:rotary_dim] = b * c + a * s
        x[:, heads:] *= k_scale
        return x.reshape(T, 2 * heads * dim)

    def retention_scan(self, qk, u, v_col, state, decay, q_indptr, slots, heads, dim, vdim, chunked=None):
        T = u.shape[0]
        q = qk[:, : heads * dim].reshape(T, heads, dim)
        k = qk[:, heads * dim :].reshape(T, heads, dim)
        v = u[:, v_col : v_col + heads * vdim].float().reshape(T, heads, vdim)
        out = torch.zeros(T, heads * vdim, dtype=torch.float32)
        for row in range(slots.numel()):
            lo, hi = int(q_indptr[row]), int(q_indptr[row + 1])
            S = state[int(slots[row])].view(heads, dim, vdim)
            for t in range(lo, hi):
                S.copy_(decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :])
                out[t] = torch.einsum("hdv,hd->hv", S, q[t]).reshape(-1)
        return out

    # ---- attention with sigmoid weights
    def sigmoid_attention_prepare(self, qkv, k_pool, v_pool, q_w, k_w, positions, slot_mapping, heads, kv_heads, dim, vdim, eps, temp_coef, temp_every,
                                  page_size):
        T = qkv.shape[0]
        Q, K = heads * dim, kv_heads * dim

        def norm(x, w):
            return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.float()

        temp = 1.0 + temp_coef * torch.log((torch.div(positions.clamp(min=0) + 1, temp_every, rounding_mode="floor") + 1).float())
        q = (norm(qkv[:, :Q].float().reshape(T, heads, dim), q_w) * temp[:, None, None]).to(qkv.dtype)
        k = norm(qkv[:, Q : Q + K].float().reshape(T, kv_heads, dim), k_w).to(qkv.dtype)
        v = qkv[:, Q + K : Q + K + kv_heads * vdim].reshape(T, kv_heads, vdim)
        for t in range(T):
            slot = int(slot_mapping[t])
            if slot < 0:
                continue
            page, off = divmod(slot, page_size)
            if v_pool is None:
                k_pool[page, :, off, :dim] = k[t]
                k_pool[page, :, off, dim:] = v[t]
            else:
                k_pool[page, :, off, :] = k[t]
                v_pool[page, :, off, :] = v[t]
        return q.contiguous()

    def sigmoid_attention(self, q, k_pool, v_pool, gate_rows, gate_col, slopes, head_bias, positions, token_row, kv_indptr, kv_indices, kv_heads, vdim,
                          scale, kv_cap=0):
        T, heads, dim = q.shape
        page_size = k_pool.shape[2]
        out = torch.zeros(T, heads * vdim, dtype=q.dtype)
        group = heads // kv_heads
        for t in range(T):
            pos = int(positions[t])
            if pos < 0:
                continue
            r = int(token_row[t])
            pages = kv_indices[int(kv_indptr[r]) : int(kv_indptr[r + 1])].long()[: pos // page_size + 1]
            assert (pages >= 0).all(), "a page the query sees was given back"
            entries = k_pool[pages].permute(1, 0, 2, 3).reshape(kv_heads, -1, k_pool.shape[3])[:, : pos + 1].float()
            keys = entries[..., :dim]
            vals = entries[..., dim:] if v_pool is None else v_pool[pages].permute(1, 0, 2, 3).reshape(kv_heads, -1, vdim)[:, : pos + 1].float()
            distance = (pos - torch.arange(pos + 1)).float()
            for h in range(heads):
                s = (keys[h // group] @ q[t, h].float()) * scale - slopes[h] * distance + head_bias[h]
                o = torch.sigmoid(s) @ vals[h // group]
                if gate_col is not None:
                    o = o * torch.sigmoid(gate_rows[t, gate_col + h * vdim : gate_col + (h + 1) * vdim].float())
                out[t, h * vdim : (h + 1) * vdim] = o.to(q.dtype)
        return out

    # ---- activations, gates, scaled sums
    def xielu(self, x, a_pos, a_neg):
        z = x.float()
        zn = torch.clamp(z, max=0.0)
        return torch.where(z > 0, a_pos * z * z + 0.5 * z, a_neg * (torch.expm1(zn) - zn) + 0.5 * zn).to(x.dtype)

    def head_gate_mul_(self, x, g, col, heads):
        T, V = x.shape
        gate = torch.sigmoid(g[:, col : col + heads].float())
        x.copy_((x.float().reshape(T, heads, V // heads) * gate[:, :, None]).reshape(T, V).to(x.dtype))
        return x

    def wide_rms_norm_gated(self, stream, w, eps, out_dtype, addend, gate, gate_bias, rows=None):
        s = stream + addend.float() * torch.sigmoid(gate + gate_bias)
        if rows is None:
            stream.copy_(s)
        else:
            s = s[rows.long()]
        if w is None:
            return s.to(out_dtype)
        return (s * torch.rsqrt((s * s).mean(-1, keepdim=True) + eps) * w).to(out_dtype)

    def scale_(self, x, factor):
        return x.mul_(factor)

    # ---- the selective scan
    def mamba1_scan(self, xc, dt, dbc, xz, dt_bias, a, d, state, q_indptr, slots, inner, N, R):
        T = xc.shape[0]
        out = torch.zeros(T, inner, dtype=xc.dtype)
        for r in range(slots.numel()):
            lo, hi = int(q_indptr[r]), int(q_indptr[r + 1])
            S = state[int(slots[r]), : inner * N].reshape(inner, N)
            for t in range(lo, hi):
                zdt = dt[t].float() + dt_bias
                step = torch.where(zdt > 20.0, zdt, torch.log1p(torch.exp(torch.clamp(zdt, max=20.0))))
                x = xc[t].float()
                B, C = dbc[t, R : R + N].float(), dbc[t, R + N : R + 2 * N].float()
                S.copy_(torch.exp(step[:, None] * a) * S + (step * x)[:, None] * B[None, :])
                y = S @ C + d * x
                z = xz[t, inner:].float()
                out[t] = (y * z / (1 + torch.exp(-z))).to(xc.dtype)
        return out

    def moe_combine(self, ys, route, shared=None):
        T = ys.shape[0] // route.top
        out = ys[route.inverse.long()].float().reshape(T, route.top, -1).sum(1)
        if shared is not None:
            out = out + shared.float()
        return out.to(ys.dtype)

    def gemm_stream_supported(self, *a):
        return False

    def gemm_stream_swiglu_supported(self, *a):
        return False

    def gemm_simt(self, a, w, out_dtype=None):
        return (a.float() @ w.float().t()).to(out_dtype or a.dtype)

    def argmax(self, logits):
        return torch.tensor([plain.sample_row(r.tolist(), 0.0) for r in logits], dtype=torch.int32)

    def sample_penalise(self, logits, counts, prompt_bits, row_slot, repetition, presence, frequency, mask_bits=None):
        out = logits.clone()
        V = logits.shape[1]
        for r in range(logits.shape[0]):
            slot = int(row_slot[r])
            if slot < 0:
                continue
            c = {v: int(n) for v, n in enumerate(counts[slot].tolist()) if n}
            words = prompt_bits[slot].tolist()
            prompt = [v for v in range(V) if (words[v >> 5] >> (v & 31)) & 1]
            out[r] = torch.tensor(plain.penalise_row(logits[r].tolist(), c, prompt, float(repetition[r]), float(frequency[r]), float(presence[r])))
            if mask_bits is not None:
                allowed = mask_bits[slot].tolist()
                for v in range(V):
                    if not (allowed[v >> 5] >> (v & 31)) & 1:
                        out[r, v] = float("-inf")
        return out

    def sample_count_tokens(self, counts, row_slot, ids):
        for r in range(ids.numel()):
            if int(row_slot[r]) >= 0 and 0 <= int(ids[r]) < counts.shape[1]:
                counts[int(row_slot[r]), int(ids[r])] += 1

    def sample_prompt_bits(self, bits_of_slot, ids):
        for v in ids.tolist():
            if 0 <= v < bits_of_slot.numel() * 32:
                word = int(bits_of_slot[v >> 5]) & 0xffffffff
                word |= 1 << (v & 31)
                bits_of_slot[v >> 5] = word - (1 << 32) if word >= (1 << 31) else word

    def sample_logprobs(self, logits, ids, top=0):
        lp = torch.tensor([plain.logprob_at(logits[r].tolist(), int(ids[r])) for r in range(logits.shape[0])], dtype=torch.float32)
        pairs = [plain.top_logprobs(logits[r].tolist(), top) for r in range(logits.shape[0])]
        R = logits.shape[0]
        return (lp, torch.tensor([p[0] for p in pairs], dtype=torch.int32).reshape(R, top),
                torch.tensor([p[1] for p in pairs], dtype=torch.float32).reshape(R, top))

    def sample(self, logits, temperature, top_k, top_p, min_p, seeds, offsets, workspace=None):
        out = []
        for r in range(logits.shape[0]):
            out.append(plain.sample_row(logits[r].tolist(), float(temperature[r]), int(top_k[r]), float(top_p[r]), float(min_p[r]),
                                        int(seeds[r]) & ((1 << 64) - 1), int(offsets[r])))
        return torch.tensor(out, dtype=torch.int32)
