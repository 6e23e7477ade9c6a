"""Plain torch versions of every kernel, with the call signatures of ``CudaKernels``.

Two uses, both in tests only: (1) the reference each CUDA kernel is compared
with on the GPU; (2) a stand-in that lets the step function, the cache manager
and the scheduler be exercised on a machine without a GPU. It is not a product
path: the engine itself has no CPU fallback. All arithmetic is float32 (float64
if asked), outputs are rounded once to the output tensor's dtype.
"""
from __future__ import annotations

import torch


class EmuKernels:
    def __init__(self, device="cpu", math_dtype=torch.float32):
        self.device = torch.device(device)
        self.math = math_dtype
        self.launches = 0

    @staticmethod
    def check_attention_shape(heads, kv_heads, head_dim):
        if head_dim % 2 or heads % kv_heads:
            raise ValueError("bad attention shape")

    def check_errors(self):
        return None

    def on_current_stream(self):
        import contextlib

        return contextlib.nullcontext()

    def fetch_ints(self, host, dev, n):
        dev.view(-1)[:n].copy_(host.view(-1)[:n])

    @staticmethod
    def _ids(tokens, last_token):
        ids = tokens.long()
        if last_token is not None:
            neg = ids < 0
            ids = torch.where(neg, last_token.long()[(-ids - 1).clamp(min=0)], ids)
        return ids

    def embedding(self, tokens, table, out, last_token=None, scale=1.0):
        out.copy_((table[self._ids(tokens, last_token)].to(torch.float32) * scale).to(out.dtype))

    def embedding_pair(self, ctx, table, pairs, state, buckets, mul_prev, mul_cur, out, scale=1.0):
        ids = self._ids(ctx.tokens, getattr(ctx, "last_token", None))
        cu, pos = ctx.cu_q.tolist(), ctx.positions.tolist()
        held = state.view(torch.int32)
        rows = []
        for r, slot in enumerate(ctx.slots.tolist()):
            for t in range(cu[r], cu[r + 1]):
                prev = int(ids[t - 1]) if t > cu[r] else int(held[slot, 0])
                rows.append(buckets if pos[t] == 0 else (prev * mul_prev + int(ids[t]) * mul_cur) % buckets)
            if cu[r + 1] > cu[r]:
                held[slot, 0] = int(ids[cu[r + 1] - 1])
        rows = torch.tensor(rows, dtype=torch.long, device=out.device)
        out.copy_((table[ids].to(torch.float32) * scale + pairs[rows].to(torch.float32)).to(out.dtype))

    def bias_round(self, sums, bias, out):
        out.copy_((sums if bias is None else sums + bias.to(sums.dtype)).to(out.dtype))

    def sigmoid_gate(self, a, gate, out, scale=1.0):
        v = a.to(self.math) * scale
        if gate is not None:
            v = v * torch.sigmoid(gate.to(self.math)).repeat_interleave(a.shape[1] // gate.shape[1], 1)
        out.copy_(v.to(out.dtype))

    def softcap(self, x, cap):
        x.copy_(cap * torch.tanh(x / cap))

    def _layer_norm(self, v, weight, eps):
        v = v.to(self.math)
        d = v - v.mean(-1, keepdim=True)
        return d * torch.rsqrt(d.pow(2).mean(-1, keepdim=True) + eps) * weight.to(self.math)

    def add_layernorm(self, x, delta, weight, eps, out):
        if delta is not None:
            x.add_(delta.to(x.dtype))
        out.copy_(self._layer_norm(x, weight, eps).to(out.dtype))

    def add_layernorm_rows(self, x, delta, rows, weight, eps, out):
        v = x[rows.long()]
        if delta is not None:
            v = v + delta[rows.long()].to(x.dtype)
        out.copy_(self._layer_norm(v, weight, eps).to(out.dtype))

    def _norm(self, v, weight, eps):
        v = v.to(self.math)
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * weight.to(self.math)

    def add_rmsnorm(self, x, delta, weight, eps, out):
        if delta is not None:
            x.add_(delta.to(x.dtype))
        out.copy_(self._norm(x, weight, eps).to(out.dtype))

    def add2_rmsnorm(self, x, delta, delta2, rows, weight, eps, out):
        if rows is None:
            x.add_(delta.to(x.dtype)).add_(delta2.to(x.dtype))
            out.copy_(self._norm(x, weight, eps).to(out.dtype))
        else:
            v = x[rows.long()] + delta[rows.long()].to(x.dtype) + delta2[rows.long()].to(x.dtype)
            out.copy_(self._norm(v, weight, eps).to(out.dtype))

    def add_rmsnorm_rows(self, x, delta, rows, weight, eps, out):
        v = x[rows.long()]
        if delta is not None:
            v = v + delta[rows.long()].to(x.dtype)
        out.copy_(self._norm(v, weight, eps).to(out.dtype))

    def linear(self, a, w, out):
        out.copy_((a.to(self.math) @ w.to(self.math).T).to(out.dtype))

    def swiglu(self, gate_up, out):
        inter = out.shape[1]
        g = gate_up[:, :inter].to(self.math)
        u = gate_up[:, inter:].to(self.math)
        out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))

    def gate_up_swiglu(self, h, w_gate_up, out):
        gate_up = torch.empty((h.shape[0], w_gate_up.shape[0]), dtype=h.dtype, device=h.device)
        self.linear(h, w_gate_up, gate_up)
        self.swiglu(gate_up, out)

    def qkv_rope_cache(self, h, w_qkv, qkv, positions, token_row, inv_freq, pairing, rotary_dim, heads, kv_heads, head_dim,
                       k_cache, v_cache, block_table, page_size, write_cache, memo=None):
        self.linear(h, w_qkv, qkv)
        self.rope_cache_write(qkv, positions, token_row, inv_freq, pairing, rotary_dim, heads, kv_heads, head_dim,
                              k_cache, v_cache, block_table, page_size, write_cache)

    def rope_cache_write(self, qkv, positions, token_row, inv_freq, pairing, rotary_dim, heads, kv_heads, head_dim,
                         k_cache, v_cache, block_table, page_size, write_cache):
        t = qkv.shape[0]
        d = head_dim
        x = qkv.view(t, heads + 2 * kv_heads, d)
        qk = x[:, : heads + kv_heads].to(self.math)
        if rotary_dim > 0:
            ang = positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, : rotary_dim // 2]
            cos, sin = ang.cos().to(self.math)[:, None, :], ang.sin().to(self.math)[:, None, :]
            if pairing == 0:
                a, b = qk[..., : rotary_dim // 2], qk[..., rotary_dim // 2: rotary_dim]
                rot = torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
            else:
                a, b = qk[..., 0:rotary_dim:2], qk[..., 1:rotary_dim:2]
                rot = torch.stack([a * cos - b * sin, b * cos + a * sin], -1).flatten(-2)
            qk = torch.cat([rot, qk[..., rotary_dim:]], -1)
        qk = qk.to(qkv.dtype)
        x[:, :heads] = qk[:, :heads]
        if write_cache:
            pos = positions.long()
            pages = block_table.long()[token_row.long(), pos // page_size]
            assert bool((pages >= 0).all()), "cache write to a missing page"
            k_cache[pages, :, pos % page_size] = qk[:, heads:]          # caches are [pages, kv_heads, page_size, D]
            v_cache[pages, :, pos % page_size] = x[:, heads + kv_heads:]

    def gate_up_activation(self, h, w_gate_up, out, activation, limit=0.0, alpha=1.0):
        gate_up = torch.empty((h.shape[0], w_gate_up.shape[0]), dtype=h.dtype, device=h.device)
        self.linear(h, w_gate_up, gate_up)
        inter = out.shape[1]
        g, u = gate_up[:, :inter].to(self.math), gate_up[:, inter:].to(self.math)
        if activation == "clamped_swish":
            g, u = torch.clamp(g, max=limit), torch.clamp(u, -limit, limit)
            out.copy_((g * torch.sigmoid(alpha * g) * (u + 1)).to(out.dtype))
        elif activation == "gelu_tanh":
            out.copy_((torch.nn.functional.gelu(g, approximate="tanh") * u).to(out.dtype))
        else:
            out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))

    def add_dynamic_tanh(self, x, delta, through, rows, params, out):
        """x += [tanh(alpha' delta) w' + b'] (``through`` = [w' | b' | alpha'], or the plain delta); out = tanh(alpha x) w + b
        with params = [w | b | alpha]; with ``rows`` only for those rows and without updating x; with x None the norm of delta."""
        def dyt(v, par):
            n = (par.shape[0] - 1) // 2
            par = par.to(self.math)
            return torch.tanh(par[2 * n] * v) * par[:n] + par[n: 2 * n]

        d = None
        if delta is not None:
            d = delta.to(self.math)
            if through is not None and x is not None:
                d = dyt(d, through).to(torch.float32)
        if x is None:
            out.copy_(dyt(d, params).to(out.dtype))
            return
        if rows is not None:
            v = x[rows.long()]
            if d is not None:
                v = v + d[rows.long()].to(x.dtype)
        else:
            if d is not None:
                x.add_(d.to(x.dtype))
            v = x
        out.copy_(dyt(v.to(self.math), params).to(out.dtype))

    def token_shift_mix(self, x, mu, state, ctx, out):
        cu = ctx.cu_q.tolist()
        for r, slot in enumerate(ctx.slots.tolist()):
            a, b = cu[r], cu[r + 1]
            if b == a:
                continue
            cur = x[a:b].to(self.math)
            prev = torch.cat([state[slot].to(self.math), cur[:-1]], 0)
            out[:, a:b] = (cur[None] + (prev - cur)[None] * mu.to(self.math)[:, None, :]).to(out.dtype)
            state[slot] = cur[-1:].to(state.dtype)

    def activation(self, x, out, kind):
        v = x.to(self.math)
        if kind == "relu_squared":
            v = torch.relu(v) ** 2
        elif kind == "tanh":
            v = torch.tanh(v)
        elif kind == "silu":
            v = v * torch.sigmoid(v)
        elif kind == "gelu_tanh":
            v = 0.5 * v * (1 + torch.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3)))
        else:
            raise ValueError(kind)
        out.copy_(v.to(out.dtype))

    def linear_activation(self, h, w, out, kind):
        self.activation(h.to(self.math) @ w.to(self.math).T, out, kind)

    def add_bias(self, x, bias):
        x.add_(bias.to(x.dtype))

    def qk_prepare(self, sums, bias, positions, token_row, heads, kv_heads, head_dim, dim, q_weight, k_weight, eps, inv_freq, rot_dims,
                   q_out, k_cache, v_cache, block_table, page_size, head_norm=False):
        t, d, m = sums.shape[0], head_dim, self.math
        x = sums[:, : (heads + 2 * kv_heads) * d].to(m)      # (the row may go on with columns that are not the kernel's)
        if bias is not None:
            x = x + bias.to(m)
        x = x.reshape(t, heads + 2 * kv_heads, d)
        ang = positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, : rot_dims // 2]
        cos, sin = ang.cos().to(m)[:, None, :], ang.sin().to(m)[:, None, :]

        def prepare(v, n_heads, weight):
            v = v.reshape(t, n_heads * d)
            if weight is not None:
                v = v * torch.rsqrt(v.pow(2).sum(-1, keepdim=True) / (n_heads * dim) + eps) * weight.to(m)
            v = v.view(t, n_heads, d).clone()
            half = rot_dims // 2
            if half:
                a, b = v[..., :half].clone(), v[..., half: rot_dims].clone()
                v[..., :half] = a * cos - b * sin
                v[..., half: rot_dims] = b * cos + a * sin
            if head_norm:
                v = v * torch.rsqrt(v.pow(2).sum(-1, keepdim=True) / dim + eps)
            return v

        q_out.copy_(prepare(x[:, :heads], heads, q_weight).reshape(t, heads * d).to(q_out.dtype))
        if kv_heads:
            self._write_pages(k_cache, prepare(x[:, heads: heads + kv_heads], kv_heads, k_weight), positions, token_row, block_table, page_size)
            self._write_pages(v_cache, x[:, heads + kv_heads:], positions, token_row, block_table, page_size)

    def linear_batched(self, a, w, out):
        """out[:, b] = a[:, b] @ w[b]^T for every b: a [M, B, K], w [B, N, K], out [M, B, N] (views with any row strides)."""
        out.copy_(torch.einsum("mbk,bnk->mbn", a.to(self.math), w.to(self.math)).to(out.dtype))

    def _write_pages(self, cache, rows, positions, token_row, block_table, page_size):
        pos = positions.long()
        pages = block_table.long()[token_row.long(), pos // page_size]
        assert bool((pages >= 0).all()), "cache write to a missing page"
        cache[pages, :, pos % page_size] = rows.to(cache.dtype)

    def normed_qk_cache_write(self, proj, positions, token_row, heads, kv_heads, head_dim, dim, q_weight, k_weight, eps, temp_coef,
                              temp_every, k_cache, v_cache, block_table, page_size, write_cache):
        t, d, m = proj.shape[0], head_dim, self.math
        x = proj.view(t, heads + 2 * kv_heads, d)
        q, k = x[:, :heads].to(m).reshape(t, heads * d), x[:, heads: heads + kv_heads].to(m).reshape(t, kv_heads * d)
        if q_weight is not None:
            q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) / (heads * dim) + eps) * q_weight.to(m)
            k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) / (kv_heads * dim) + eps) * k_weight.to(m)
        if temp_coef:
            temp = 1.0 + temp_coef * torch.log((torch.div(positions.long() + 1, temp_every, rounding_mode="floor") + 1).to(torch.float32))
            q = q * temp.to(m)[:, None]
        x[:, :heads] = q.view(t, heads, d).to(proj.dtype)
        if write_cache:
            self._write_pages(k_cache, k.view(t, kv_heads, d), positions, token_row, block_table, page_size)
            self._write_pages(v_cache, x[:, heads + kv_heads:], positions, token_row, block_table, page_size)

    def latent_prepare(self, proj, n_q, positions, token_row, c_weight, eps, inv_freq, rot_dims, heads, dim, rot_dim, rank, head_dim,
                       q_lat, k_cache, block_table, page_size, write_cache, q_off=None, row_out=None, half_pairs=False,
                       latent=None):
        t, m = proj.shape[0], self.math
        ang = positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, :]
        cos, sin = ang.cos().to(m), ang.sin().to(m)

        def rotate(v):                      # [..., rot_dim] with t leading
            shape = (t,) + (1,) * (v.dim() - 2) + (rot_dims // 2,)
            c, s = cos.view(shape), sin.view(shape)
            if half_pairs:
                a, b = v[..., : rot_dims // 2], v[..., rot_dims // 2: rot_dims]
                return torch.cat([a * c - b * s, b * c + a * s, v[..., rot_dims:]], -1)
            a, b = v[..., 0:rot_dims:2], v[..., 1:rot_dims:2]
            return torch.cat([torch.stack([a * c - b * s, b * c + a * s], -1).flatten(-2), v[..., rot_dims:]], -1)

        q = proj[:, :n_q].view(t, heads, dim + rot_dim).to(m)
        q_off = rank if q_off is None else q_off
        ql = q_lat[:, : heads * head_dim].view(t, heads, head_dim)
        ql[:, :, q_off: q_off + rot_dim] = rotate(q[..., dim:]).to(q_lat.dtype)
        ql[:, :, q_off + rot_dim:] = 0
        down = (proj[:, n_q: n_q + rank + rot_dim] if latent is None else latent[:, : rank + rot_dim]).to(m)
        c = down[:, :rank]
        c = c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps) * c_weight.to(m)
        if row_out is not None:
            row_out[:, :rank] = c.to(row_out.dtype)
            row_out[:, rank: rank + rot_dim] = rotate(down[:, rank:]).to(row_out.dtype)
        if write_cache:
            row = torch.zeros((t, 1, head_dim), dtype=m, device=proj.device)
            row[:, 0, :rank] = c
            row[:, 0, rank: rank + rot_dim] = rotate(down[:, rank:])
            self._write_pages(k_cache, row, positions, token_row, block_table, page_size)

    def table_experts(self, h, tokens, last_token, table, w_up, w_down, top, out, activation="relu_squared"):
        m = self.math
        idx = table.long()[self._ids(tokens, last_token)]            # [T, top]
        total = torch.zeros((h.shape[0], w_down.shape[1]), dtype=m, device=h.device)
        for slot in range(top):
            for e in idx[:, slot].unique().tolist():
                rows = (idx[:, slot] == e).nonzero().flatten()
                a = torch.relu(h[rows].to(m) @ w_up[e].to(m).T) ** 2
                total[rows] += (a.to(h.dtype).to(m) @ w_down[e].to(m).T) / top
        out.copy_(total.to(out.dtype))

    def attention(self, qkv, k_cache, v_cache, block_table, cu_q, kv_len, token_row, positions, heads, kv_heads, head_dim,
                  page_size, scale, window, out, shape, slopes=None, chunk=0, softcap=0.0, sinks=None, keep_first=0):
        d = head_dim
        g = heads // kv_heads
        cu = cu_q.tolist()
        lens = kv_len.tolist()
        for r in range(len(lens)):
            q0, q1 = cu[r], cu[r + 1]
            n, L = q1 - q0, lens[r]
            if n == 0:
                continue
            q = qkv[q0:q1, : heads * d].view(n, heads, d).to(self.math)
            key_pos = torch.arange(L, device=qkv.device)
            lo = max(0, (L - n) - window + 1) if window else 0
            if chunk:
                lo = max(lo, ((L - n) // chunk) * chunk)
            keys = key_pos[lo:]
            if window and keep_first and lo > 0:
                keys = torch.cat([key_pos[: min(keep_first, lo)], keys])       # the first tokens stay readable behind the window
            pages = block_table[r].long()[keys // page_size]
            assert bool((pages >= 0).all()), "attention reads a missing page"
            k = k_cache[pages, :, keys % page_size].to(self.math)
            v = v_cache[pages, :, keys % page_size].to(self.math)
            kk, vv = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
            s = torch.einsum("thd,shd->hts", q, kk) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)       # before any distance bias
            qp = torch.arange(L - n, L, device=qkv.device)[:, None]
            kp = keys[None, :]
            mask = kp > qp
            if window:
                mask = mask | ((kp <= qp - window) & (kp >= keep_first))
            if chunk:
                mask = mask | (kp < (qp // chunk) * chunk)
            if slopes is not None:
                s = s - slopes.to(self.math)[:, None, None] * (qp - kp).to(self.math)[None]
            s = s.masked_fill(mask[None], float("-inf"))
            if sinks is not None:
                # the sink is one more score without a value: a column that the product with the values leaves out
                s = torch.cat([s, sinks.to(self.math)[:, None, None].expand(heads, n, 1)], -1)
                o = torch.einsum("hts,shd->thd", torch.softmax(s, -1)[..., :-1], vv)
            else:
                o = torch.einsum("hts,shd->thd", torch.softmax(s, -1), vv)
            out[q0:q1] = o.reshape(n, heads * d).to(out.dtype)

    # ---- mixers with recurrent state, routed experts -------------------------------------------------------------
    def causal_conv(self, x, weight, bias, state, ctx, out, activation="none", residual=False):
        taps = weight.shape[1]
        k = taps - 1
        cu = ctx.cu_q.tolist()
        w = weight.to(self.math)
        for r, slot in enumerate(ctx.slots.tolist()):
            a, b = cu[r], cu[r + 1]
            seq = x[a:b].to(self.math) if not k else torch.cat([state[slot].to(self.math), x[a:b].to(self.math)], 0)   # [k + n, C]
            acc = torch.zeros((b - a, x.shape[1]), dtype=self.math, device=x.device)
            for j in range(taps):
                acc = acc + seq[j: j + b - a] * w[:, j]
            if bias is not None:
                acc = acc + bias.to(self.math)
            if residual:
                acc = acc + x[a:b].to(self.math)
            if activation == "silu":
                acc = acc * torch.sigmoid(acc)
            out[a:b] = acc.to(out.dtype)
            if k:
                state[slot] = seq[-k:].to(state.dtype)

    def linear_recurrence(self, mode, q, k, v, state, ctx, out, heads, qk_heads, dk, dv, aux=None, rate=None, decay=None,
                          a_log=None, dt_bias=None, d_skip=None, q_scale=1.0, rate_per_head=False, bonus=None, rate_scale=1.0):
        m = self.math
        f = torch.nn.functional
        cu = ctx.cu_q.tolist()
        rep = heads // qk_heads
        for r, slot in enumerate(ctx.slots.tolist()):
            a, b = cu[r], cu[r + 1]
            n = b - a
            qq = q[a:b, : qk_heads * dk].to(m).reshape(n, qk_heads, dk).repeat_interleave(rep, 1)
            kk = k[a:b, : qk_heads * dk].to(m).reshape(n, qk_heads, dk).repeat_interleave(rep, 1)
            vv = v[a:b, : heads * dv].to(m).reshape(n, heads, dv)
            s = state[slot].to(m)                                                            # [heads, dk, dv]
            if mode == "decay":
                qq, kk, vv = f.silu(qq), f.silu(kk), f.silu(vv)
                dec = decay.to(m)[None, :, None].expand(n, heads, dk)
                u_scale = torch.ones(n, heads, dtype=m, device=q.device)
            elif mode == "ssm":
                dt = f.softplus(aux[a:b, :heads].to(m) + dt_bias.to(m), threshold=20.0)
                dec = torch.exp(-torch.exp(a_log.to(m)) * dt)[:, :, None].expand(n, heads, dk)
                u_scale = dt
            elif mode == "wkv":
                dec = torch.exp(-torch.exp(rate[a:b, : heads * dk].to(m) + dt_bias.to(m))).reshape(n, heads, dk)
                extra = bonus.to(m).reshape(heads, dk)
            elif mode == "gla":
                qq = qq * q_scale
                dec = torch.exp(f.logsigmoid(rate[a:b, : heads * dk].to(m) + dt_bias.to(m)) * rate_scale).reshape(n, heads, dk)
                u_scale = torch.ones(n, heads, dtype=m, device=q.device)
            else:
                qq = qq / torch.sqrt((qq * qq).sum(-1, keepdim=True) + 1e-6) * q_scale
                kk = kk / torch.sqrt((kk * kk).sum(-1, keepdim=True) + 1e-6)
                cols = heads if rate_per_head else heads * dk
                rr = f.softplus(rate[a:b, :cols].to(m) + dt_bias.to(m), threshold=20.0).reshape(n, heads, -1).expand(n, heads, dk)
                dec = torch.exp(-torch.exp(a_log.to(m))[None, :, None] * rr)
                beta = torch.sigmoid(aux[a:b, :heads].to(m))
            for i in range(n):
                if mode == "wkv":
                    # the read-out sees the state before this token, and this token's own k v^T times the bonus
                    o = torch.einsum("hkv,hk->hv", s, qq[i]) + (extra * kk[i] * qq[i]).sum(-1, keepdim=True) * vv[i]
                    s = s * dec[i][:, :, None] + kk[i][:, :, None] * vv[i][:, None, :]
                    out[a + i] = o.reshape(-1).to(out.dtype)
                    continue
                s = s * dec[i][:, :, None]
                if mode == "delta":
                    u = beta[i][:, None] * (vv[i] - torch.einsum("hkv,hk->hv", s, kk[i]))
                else:
                    u = u_scale[i][:, None] * vv[i]
                s = s + kk[i][:, :, None] * u[:, None, :]
                o = torch.einsum("hkv,hk->hv", s, qq[i])
                if mode == "ssm":
                    o = o + d_skip.to(m)[:, None] * vv[i]
                out[a + i] = o.reshape(-1).to(out.dtype)
            state[slot] = s.to(state.dtype)

    def gated_norm(self, y, out, groups=0, eps=0.0, weight=None, gate=None, gate_act="sigmoid", gate_first=False, scale=1.0):
        m = self.math
        v = y.to(m)
        t, c = v.shape
        g = None
        if gate is not None:
            g = gate.to(m)
            g = g * torch.sigmoid(g) if gate_act == "silu" else torch.sigmoid(g)
            g = g.repeat_interleave(c // gate.shape[1], 1)
        if g is not None and gate_first:
            v = v * g
        if groups:
            v = v.reshape(t, groups, c // groups)
            v = (v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)).reshape(t, c)
        if weight is not None:
            v = v * weight.to(m).repeat(c // weight.shape[0])
        if g is not None and not gate_first:
            v = v * g
        out.copy_((v * scale).to(out.dtype))

    def kv_norm_cache_write(self, qkv, positions, token_row, heads, kv_heads, head_dim, norm_dim, eps, k_cache, v_cache, block_table,
                            page_size):
        t, d = qkv.shape[0], head_dim
        x = qkv[:, : (heads + 2 * kv_heads) * d].reshape(t, heads + 2 * kv_heads, d)
        kk, vv = x[:, heads: heads + kv_heads], x[:, heads + kv_heads:].to(self.math)
        if norm_dim:
            vv = vv / torch.sqrt((vv[..., :norm_dim] ** 2).mean(-1, keepdim=True) + eps)
        pos = positions.long()
        pages = block_table.long()[token_row.long(), pos // page_size]
        assert bool((pages >= 0).all()), "cache write to a missing page"
        k_cache[pages, :, pos % page_size] = kk
        v_cache[pages, :, pos % page_size] = vv.to(v_cache.dtype)

    def routed_experts(self, h, logits, w_gate_up, w_down, top, out, score="sigmoid", renormalise=False, scale_input=True,
                       activation="clamped_swish", limit=0.0, alpha=1.702, outputs=None, choice_bias=None, renormalise_eps=0.0,
                       shared=None, shared_gated=False, weight_scale=1.0):
        m = self.math
        n_out = logits.shape[1] if outputs is None else outputs
        z = logits[:, :n_out].to(torch.float32)
        scores = torch.sigmoid(z) if score == "sigmoid" else torch.softmax(z, -1)
        if choice_bias is not None:
            idx = torch.topk(scores + choice_bias.to(torch.float32), top, dim=-1).indices
        else:
            idx = torch.topk(z, top, dim=-1).indices             # by logit: scores of large logits round to ties
        wts = torch.gather(scores, 1, idx)
        if renormalise:
            wts = wts / (wts.sum(-1, keepdim=True) + renormalise_eps)
        wts = wts * weight_scale
        ff = w_down.shape[2]
        n_real = w_down.shape[0]
        total = torch.zeros((h.shape[0], w_down.shape[1]), dtype=m, device=h.device)
        if shared is not None:
            g = torch.sigmoid(logits[:, n_out: n_out + 1].to(m)) if shared_gated else 1.0
            total += g * shared.to(m)
        for slot in range(top):
            for e in idx[:, slot].unique().tolist():
                rows = (idx[:, slot] == e).nonzero().flatten()
                w = wts[rows, slot].to(m)[:, None]
                if e >= n_real:                                  # an identity expert: the token's input itself
                    total[rows] += h[rows].to(m) * w
                    continue
                gu = h[rows].to(m) @ w_gate_up[e].to(m).T
                if scale_input:
                    gu = gu * w
                g, u = gu[:, :ff], gu[:, ff:]
                if activation == "clamped_swish":
                    g, u = torch.clamp(g, max=limit), torch.clamp(u, -limit, limit)
                    a = g * torch.sigmoid(alpha * g) * (u + 1)
                else:
                    a = g * torch.sigmoid(g) * u
                y = a.to(h.dtype).to(m) @ w_down[e].to(m).T
                total[rows] += y if scale_input else y * w
        out.copy_(total.to(out.dtype))

    def sample(self, logits, temperature, req_ids, tok_index, seed, out, slots=None, last_token=None):
        from tests.plain.llama_plain import sample_token

        for r in range(logits.shape[0]):
            out[r] = sample_token(logits[r], float(temperature[r]), seed, int(req_ids[r]), int(tok_index[r]))
            if slots is not None and last_token is not None:
                last_token[int(slots[r])] = out[r]
