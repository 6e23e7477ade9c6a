"""Latent attention: keys and values are read out of one small vector per token.

Per token: q = W_q h, laid out head by head as [dim plain | rot_dim rotated]; W_dkv h has kv_rank + rot_dim rows: the
first kv_rank, divided by their root mean square and multiplied by a weight, are the latent c; the last rot_dim are
one key part that all heads share and that is rotated by position (interleaved pairs (2i, 2i+1), angle = position *
base^(-2i / dims), on the first ``rot_dims`` of them), as the rot_dim part of every query head is. Head n's plain key
is U_n c (U = "uk", [heads * dim, kv_rank]) and its value V_n c ("uv"). score = (q_plain . U_n c + q_rot . k_rot) *
scale, causal, ordinary softmax.

Only c and the rotated key part are cached, one row of kv_rank + rot_dim numbers per token (rounded up to a multiple
of 16) for all heads. The products with U and V move to the query's side, where they cost once per query instead of
once per cached key: q_plain . (U_n c) = (U_n^T q_plain) . c, so the query becomes [U_n^T q_plain | q_rot] and the
attention is one over a single shared key/value head whose keys and values are the same cached rows; the attention's
output per head, sum_j p_j c_j, then goes through V_n and the output projection. Both per-head products are batched
library products. The cache's value tensor is its key tensor (``CacheNeed.shared_kv``).

With ``q_rank`` the queries come through a low-rank step of their own: c_q = W_dq h ("dq" [q_rank, hidden]) divided by its
root mean square and multiplied by a weight ("dq.norm"), then q = W_uq c_q ("uq" [heads * (dim + rot_dim), q_rank]); there
is no "q" tensor then. ``pairing`` "half" rotates pairs (i, i + rot_dims / 2) instead of neighbours.

The attention kernels' rows end at 256 numbers. A model whose kv_rank + rot_dim is larger runs the other way round: every
head's key [U_n c | rotated part] and value V_n c are read out when the token arrives and cached in ordinary pages, one
key/value head per query head (``per_head``; more cache, the same results).
"""
from __future__ import annotations

import math
import os

import torch

from .base import CacheNeed, Mixer, TensorDecl, register_part


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    """params: hidden, heads, dim, rot_dim, vdim, kv_rank, scale, rot_base, rot_dims (default rot_dim), eps, window (None), names,
    q_rank (None: queries straight from the input), pairing ("interleaved" | "half"), rot_scaling (as the rotary part's, or None),
    per_head (default: only when kv_rank + rot_dim exceeds the attention kernels' widest row)."""

    MAX_ROW = 256        # the widest head the attention kernels take

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.heads = int(p["hidden"]), int(p["heads"])
        self.dim, self.rot_dim, self.vdim, self.rank = int(p["dim"]), int(p["rot_dim"]), int(p["vdim"]), int(p["kv_rank"])
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.dim + self.rot_dim)
        self.rot_base = float(p["rot_base"])
        self.rot_dims = int(p.get("rot_dims") or self.rot_dim)
        if self.rot_dims % 2 or self.rot_dims > self.rot_dim:
            raise ValueError(f"rot_dims {self.rot_dims} must be even and at most rot_dim {self.rot_dim}")
        self.eps = float(p["eps"])
        self.q_rank = int(p["q_rank"]) if p.get("q_rank") else 0
        if p.get("pairing", "interleaved") not in ("interleaved", "half"):
            raise ValueError(f"latent_attention: pairing {p['pairing']!r} is not known (interleaved, half)")
        self.half_pairs = p.get("pairing", "interleaved") == "half"
        self.rot_scaling = p.get("rot_scaling")
        self.window = int(p["window"]) if p.get("window") else None
        self.names = dict(p.get("names", {}))
        self.row = self.rank + self.rot_dim                       # what a token leaves in the cache
        self.head_dim = 16 * -(-self.row // 16)
        # (SERVE_B200_LATENT_PER_HEAD=1: measurements of the other form at any size)
        self.per_head = bool(p.get("per_head", self.head_dim > self.MAX_ROW or os.environ.get("SERVE_B200_LATENT_PER_HEAD") == "1"))
        if self.per_head:
            self.head_dim = 16 * -(-max(self.dim + self.rot_dim, self.vdim) // 16)
            self.mixed_size = self.heads * self.head_dim
            runtime.kernels.check_attention_shape(self.heads, self.heads, self.head_dim)
        else:
            self.mixed_size = self.heads * self.vdim
            runtime.kernels.check_attention_shape(self.heads, 1, self.head_dim)

    def _name(self, key):
        return self.prefix + self.names.get(key, key)

    def kernel_needs(self):
        return {"attention_head_dims": [self.head_dim], "libraries": ["prep"] + (["seq"] if self.q_rank else [])}

    def tensor_decls(self):
        n_q = self.heads * (self.dim + self.rot_dim)
        queries = [TensorDecl(self._name("q"), (n_q, self.hidden))] if not self.q_rank else [
            TensorDecl(self._name("dq"), (self.q_rank, self.hidden)), TensorDecl(self._name("dq.norm"), (self.q_rank,), role="vector", init="norm"),
            TensorDecl(self._name("uq"), (n_q, self.q_rank))]
        return queries + [
                TensorDecl(self._name("dkv"), (self.row, self.hidden)),
                TensorDecl(self._name("dkv.norm"), (self.rank,), role="vector", init="norm"),
                TensorDecl(self._name("uk"), (self.heads * self.dim, self.rank)),
                TensorDecl(self._name("uv"), (self.heads * self.vdim, self.rank)),
                TensorDecl(self._name("o"), (self.hidden, self.heads * self.vdim))]

    def load(self, tensors):
        # one product for q and the down projection; its row count is padded to a multiple of 8 (16-byte rows in bfloat16)
        self.n_q = self.heads * (self.dim + self.rot_dim)
        if self.q_rank:
            # the input's product gives [latent | shared key part | query latent] (rows padded to a multiple of 8); the queries'
            # second step fills a buffer of its own
            w = torch.cat([tensors[self._name("dkv")], tensors[self._name("dq")]], dim=0)
            self.n_in = 8 * -(-w.shape[0] // 8)
            if self.n_in != w.shape[0]:
                w = torch.cat([w, w.new_zeros((self.n_in - w.shape[0], w.shape[1]))], dim=0)
            self.w_uq = tensors[self._name("uq")].contiguous()
            self.q_norm = tensors[self._name("dq.norm")].float().contiguous()
        else:
            w = torch.cat([tensors[self._name("q")], tensors[self._name("dkv")]], dim=0)
            self.n_in = 8 * -(-w.shape[0] // 8)
            if self.n_in != w.shape[0]:
                w = torch.cat([w, w.new_zeros((self.n_in - w.shape[0], w.shape[1]))], dim=0)
        self.w_in = w.contiguous()
        self.c_norm = tensors[self._name("dkv.norm")].float().contiguous()
        # U_n^T as the [N, K] operand of out = a @ w^T: [heads, kv_rank, dim]
        self.w_uk_t = tensors[self._name("uk")].view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[self._name("uv")].view(self.heads, self.vdim, self.rank).contiguous()
        w_o = tensors[self._name("o")]
        if self.per_head:
            self.w_uk = tensors[self._name("uk")].view(self.heads, self.dim, self.rank).contiguous()
            if self.vdim != self.head_dim:
                padded = w_o.new_zeros((self.hidden, self.heads, self.head_dim))
                padded[:, :, : self.vdim] = w_o.view(self.hidden, self.heads, self.vdim)
                w_o = padded.view(self.hidden, self.heads * self.head_dim)
        self.w_o = w_o.contiguous()
        if self.rot_scaling:
            from .rotary import rotary_inv_freq

            self.inv_freq = rotary_inv_freq(self.rot_dims, self.rot_base, self.rot_scaling).to(self.w_o.device)
        else:
            i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
            self.inv_freq = (self.rot_base ** (-2.0 * i / self.rot_dims)).to(torch.float32).to(self.w_o.device)

    def cache_need(self):
        if self.per_head:
            return CacheNeed(kv_heads=self.heads, head_dim=self.head_dim, window=self.window)
        return CacheNeed(kv_heads=1, head_dim=self.head_dim, window=self.window, shared_kv=True)

    def output_weight(self):
        return self.w_o

    def mix_into(self, h, ctx, cache, out, scale: float = 1.0):
        if scale != 1.0:
            raise ValueError("latent_attention writes its heads unscaled")
        k = self.rt.kernels
        t, d = h.shape[0], self.head_dim
        latent = None
        if self.q_rank:
            latent = self.rt.empty_act((t, self.n_in))
            k.linear(h, self.w_in, latent)
            cq = self.rt.empty_act((t, self.q_rank))
            k.gated_norm(latent[:, self.row: self.row + self.q_rank], cq, groups=1, eps=self.eps, weight=self.q_norm)
            proj = self.rt.empty_act((t, self.n_q))
            k.linear(cq, self.w_uq, proj)
        else:
            proj = self.rt.empty_act((t, self.n_in))
            k.linear(h, self.w_in, proj)
        table = ctx.block_tables[cache.group]
        more = {**({"half_pairs": True} if self.half_pairs else {}), **({"latent": latent} if latent is not None else {})}
        if self.per_head:
            return self._mix_per_head(proj, ctx, cache, table, out, more)
        q_lat = self.rt.empty_act((t, self.heads * d))             # per head [U^T q_plain | q_rot | zeros]
        k.latent_prepare(proj, self.n_q, ctx.positions, ctx.token_row, self.c_norm, self.eps, self.inv_freq, self.rot_dims, self.heads,
                         self.dim, self.rot_dim, self.rank, d, q_lat, cache.k, table, cache.page_size, cache.writes, **more)
        q3 = proj[:, : self.n_q].view(t, self.heads, self.dim + self.rot_dim)
        k.linear_batched(q3[:, :, : self.dim], self.w_uk_t, q_lat.view(t, self.heads, d)[:, :, : self.rank])
        o_lat = self.rt.empty_act((t, self.heads * d))
        k.attention(q_lat, cache.k, cache.v, table, ctx.cu_q, ctx.kv_len, ctx.token_row, ctx.positions, self.heads, 1, d,
                    cache.page_size, self.scale, self.window or 0, o_lat, ctx.shape)
        k.linear_batched(o_lat.view(t, self.heads, d)[:, :, : self.rank], self.w_uv, out.view(t, self.heads, self.vdim))

    def _mix_per_head(self, proj, ctx, cache, table, out, more):
        """Keys and values read out per head when the token arrives: qkv [T, 3 H, D] = queries [q_plain | q_rot], keys
        [U_n c | k_rot], values V_n c (zeros after each), cached like any attention's."""
        k = self.rt.kernels
        t, d, hh = proj.shape[0], self.head_dim, self.heads
        qkv = torch.zeros((t, 3 * hh * d), dtype=proj.dtype, device=proj.device)
        row = self.rt.empty_act((t, 8 * -(-self.row // 8)))
        k.latent_prepare(proj, self.n_q, ctx.positions, ctx.token_row, self.c_norm, self.eps, self.inv_freq, self.rot_dims, hh, self.dim,
                         self.rot_dim, self.rank, d, qkv, None, table, cache.page_size, False, q_off=self.dim, row_out=row, **more)
        q3 = qkv.view(t, 3 * hh, d)
        q3[:, :hh, : self.dim].copy_(proj[:, : self.n_q].view(t, hh, self.dim + self.rot_dim)[:, :, : self.dim])
        c = row[:, None, : self.rank].expand(t, hh, self.rank)
        k.linear_batched(c, self.w_uk, q3[:, hh: 2 * hh, : self.dim])
        q3[:, hh: 2 * hh, self.dim: self.dim + self.rot_dim].copy_(row[:, None, self.rank: self.row].expand(t, hh, self.rot_dim))
        k.linear_batched(c, self.w_uv, q3[:, 2 * hh:, : self.vdim])
        k.normed_qk_cache_write(qkv, ctx.positions, ctx.token_row, hh, hh, d, d, None, None, 0.0, 0.0, 1, cache.k, cache.v, table,
                                cache.page_size, cache.writes)
        k.attention(qkv, cache.k, cache.v, table, ctx.cu_q, ctx.kv_len, ctx.token_row, ctx.positions, hh, hh, d, cache.page_size,
                    self.scale, self.window or 0, out, ctx.shape)

    def forward(self, h, ctx, cache):
        mixed = self.rt.empty_act((h.shape[0], self.mixed_size))
        self.mix_into(h, ctx, cache, mixed)
        out = self.rt.empty_act((h.shape[0], self.hidden))
        self.rt.kernels.linear(mixed, self.w_o, out)
        return out
