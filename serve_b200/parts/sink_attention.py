"""Grouped-query softmax attention with rotation, a window that keeps the first tokens, and a sink.

q = W_q h (+ b_q), k = W_k h (+ b_k), v = W_v h (+ b_v). With ``qk_norm_eps`` the whole query projection of a token (all
heads at once) is divided by its root mean square and multiplied by a weight of that size ("q.norm"), and the key
projection likewise ("k.norm"), before the rotation. The position part turns the first ``rotary_dim`` elements of every
query and key head. score = (q . k) * scale. Position i reads position j <= i if i - j < window or j < keep_first; kept
tokens keep their true positions. With ``sink`` the softmax's denominator also holds exp(sink_h), a learned number per
head without key or value. With ``own_kv`` false the mixer has no key or value tensors: it reads the pages another
execution wrote (the schedule's ``cache_of``), with its own queries, mask and sink. Query/key size and value size may
differ: pages and kernels have one head size, the larger of the two rounded up to a multiple of 16, and what lies
beyond a head's true size is zero. The projection's sums stay float until bias, norm and rotation are done, so queries
and cached keys are rounded once.
"""
from __future__ import annotations

import math

import torch

from .base import CacheNeed, Mixer, TensorDecl, build_part, register_part
from .biased_attention import _pad_heads
from .rotary import PAIRING_HALF


@register_part("mixer", "rotary_sink_attention")
class RotarySinkAttention(Mixer):
    """params: hidden, heads, kv_heads, dim, vdim, scale, bias (bool), qk_norm_eps (None: no norm), sink (bool), window
    (None: all keys), keep_first, own_kv (bool), position (PartSpec), names."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.heads, self.kv_heads = int(p["hidden"]), int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        if self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.dim)
        self.bias = bool(p.get("bias", False))
        self.qk_norm_eps = float(p["qk_norm_eps"]) if p.get("qk_norm_eps") is not None else None
        self.sink = bool(p.get("sink", False))
        self.window = int(p["window"]) if p.get("window") else None
        self.keep_first = int(p.get("keep_first") or 0) if self.window else 0
        self.own_kv = bool(p.get("own_kv", True))
        self.position = build_part("position", p["position"], runtime)
        if self.position.rotary_dim > self.dim:
            raise ValueError("rotary_dim exceeds the query/key size")
        if self.position.rotary_dim and self.position.pairing != PAIRING_HALF:
            raise ValueError("rotary_sink_attention rotates pairs (i, i + rotary_dim / 2)")
        self.names = dict(p.get("names", {}))
        self.head_dim = 16 * -(-max(self.dim, self.vdim) // 16)
        self.mixed_size = self.heads * self.head_dim
        self.cached_heads = self.kv_heads if self.own_kv else 0
        runtime.kernels.check_attention_shape(self.heads, self.kv_heads, self.head_dim)

    def _name(self, key):
        return self.prefix + self.names.get(key, key)

    def kernel_needs(self):
        return {"attention_head_dims": [self.head_dim], "libraries": ["prep"]}

    def tensor_decls(self):
        sizes = [("q", self.heads * self.dim)] + ([("k", self.kv_heads * self.dim), ("v", self.kv_heads * self.vdim)] if self.own_kv else [])
        decls = [TensorDecl(self._name(n), (rows, self.hidden)) for n, rows in sizes]
        decls.append(TensorDecl(self._name("o"), (self.hidden, self.heads * self.vdim)))
        if self.bias:
            decls += [TensorDecl(self._name(n + ".b"), (rows,), role="vector", init="small") for n, rows in sizes]
            decls.append(TensorDecl(self._name("o.b"), (self.hidden,), role="vector", init="small"))
        if self.qk_norm_eps is not None:
            decls += [TensorDecl(self._name(n + ".norm"), (rows,), role="vector", init="norm") for n, rows in sizes if n != "v"]
        if self.sink:
            decls.append(TensorDecl(self._name("sink"), (self.heads,), role="vector", init="normal"))
        return decls

    def load(self, tensors):
        d = self.head_dim
        shapes = [("q", self.heads, self.dim)] + ([("k", self.kv_heads, self.dim), ("v", self.kv_heads, self.vdim)] if self.own_kv else [])
        self.w_in = torch.cat([_pad_heads(tensors[self._name(n)], h, size, d) for n, h, size in shapes], dim=0).contiguous()
        vec = lambda name, h, size: _pad_heads(tensors[self._name(name)].float().view(-1, 1), h, size, d).view(-1)
        # float vectors laid out like the padded projection: the bias of every column, the norm weight of the query and key columns
        self.b_in = torch.cat([vec(n + ".b", h, size) for n, h, size in shapes]).contiguous() if self.bias else None
        self.q_norm = self.k_norm = None
        if self.qk_norm_eps is not None:
            self.q_norm = vec("q.norm", self.heads, self.dim).contiguous()
            self.k_norm = vec("k.norm", self.kv_heads, self.dim).contiguous() if self.own_kv else None
        w_o = tensors[self._name("o")]
        if self.vdim != d:
            padded = w_o.new_zeros((self.hidden, self.heads, d))
            padded[:, :, : self.vdim] = w_o.view(self.hidden, self.heads, self.vdim)
            w_o = padded.view(self.hidden, self.heads * d)
        self.w_o = w_o.contiguous()
        self.b_o = tensors[self._name("o.b")].float().contiguous() if self.bias else None
        self.sinks = tensors[self._name("sink")].float().contiguous() if self.sink else None

    def cache_need(self):
        return CacheNeed(kv_heads=self.kv_heads, head_dim=self.head_dim, window=self.window, keep_first=self.keep_first)

    def output_weight(self):
        return self.w_o

    def mix_into(self, h, ctx, cache, out, scale: float = 1.0):
        if scale != 1.0 or not out.is_contiguous():
            raise ValueError("rotary_sink_attention writes its heads unscaled into a contiguous buffer")
        if cache.writes != self.own_kv:
            raise ValueError("an attention without key/value tensors must read another execution's cache, and one with them its own")
        k = self.rt.kernels
        t, d = h.shape[0], self.head_dim
        sums = torch.empty((t, (self.heads + 2 * self.cached_heads) * d), dtype=torch.float32, device=h.device)
        k.linear(h, self.w_in, sums)
        table = ctx.block_tables[cache.group]
        q = self.rt.empty_act((t, self.heads * d))
        k.qk_prepare(sums, self.b_in, ctx.positions, ctx.token_row, self.heads, self.cached_heads, d, self.dim, self.q_norm, self.k_norm,
                     self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, self.position.inv_freq, self.position.rotary_dim,
                     q, cache.k, cache.v, table, cache.page_size)
        k.attention(q, cache.k, cache.v, table, ctx.cu_q, ctx.kv_len, ctx.token_row, ctx.positions, self.heads, self.kv_heads, d,
                    cache.page_size, self.scale, self.window or 0, out, ctx.shape, sinks=self.sinks,
                    **({"keep_first": self.keep_first} if self.keep_first else {}))

    def forward(self, h, ctx, cache):
        mixed = self.rt.empty_act((h.shape[0], self.mixed_size))
        self.mix_into(h, ctx, cache, mixed)
        if self.b_o is None:
            out = self.rt.empty_act((h.shape[0], self.hidden))
            self.rt.kernels.linear(mixed, self.w_o, out)
            return out
        out = torch.empty((h.shape[0], self.hidden), dtype=torch.float32, device=h.device)      # float sums, so the bias joins unrounded
        self.rt.kernels.linear(mixed, self.w_o, out)
        self.rt.kernels.add_bias(out, self.b_o)
        return out
