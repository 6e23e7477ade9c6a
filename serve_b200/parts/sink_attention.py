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

More options. ``head_norm_eps``: every query and key head is divided, after its rotation, by its own root mean square
over ``dim`` elements, without a weight. ``conv`` = taps: q, k and v (bias included) each pass a short causal convolution
over time, one filter per channel ("q.conv", "k.conv", "v.conv"), before anything else; the last taps - 1 projected
values of a request are its state. ``gate``: "element" multiplies the concatenated heads element by element with
sigmoid(W_g h) ("g" [heads * vdim, hidden]), "head" multiplies head n by sigmoid(W_g h)_n ("g" [heads, hidden]); both
read the layer's input. ``out_bias`` (default: as ``bias``) says whether the output projection has a bias too.
"""
from __future__ import annotations

import math

import torch

from ..config.spec import PartSpec
from .base import CacheNeed, Mixer, TensorDecl, build_part, register_part
from .biased_attention import _pad_heads
from .rotary import PAIRING_HALF


@register_part("mixer", "rotary_sink_attention")
class RotarySinkAttention(Mixer):
    """params: hidden, heads, kv_heads, dim, vdim, scale, bias (bool), out_bias (bool), qk_norm_eps (None: no norm),
    head_norm_eps (None), conv (taps or None), gate (None | "element" | "head"), sink (bool), window (None: all keys),
    keep_first, own_kv (bool), position (PartSpec), names."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.heads, self.kv_heads = int(p["hidden"]), int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        if self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.dim)
        self.bias = bool(p.get("bias", False))
        self.out_bias = bool(p.get("out_bias", self.bias))
        self.head_norm_eps = float(p["head_norm_eps"]) if p.get("head_norm_eps") is not None else None
        self.gate = p.get("gate")
        if self.gate not in (None, "element", "head"):
            raise ValueError(f"rotary_sink_attention: gate {self.gate!r} is not known (element, head)")
        self.taps = int(p["conv"]) if p.get("conv") else 0
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
        if self.head_norm_eps is not None and self.qk_norm_eps is not None:
            raise ValueError("rotary_sink_attention: queries and keys are normalised over the projection or per head, not both")
        if self.taps and (not self.own_kv or self.qk_norm_eps is not None or self.head_norm_eps is not None or self.position.rotary_dim):
            raise ValueError("rotary_sink_attention: the convolved form has keys of its own, no norm and no rotation")
        # the gate's projection: one column per element of the padded heads, or one per head (rows padded to a multiple of 8)
        self.gate_cols = 0 if self.gate is None else (self.mixed_size if self.gate == "element" else 8 * -(-self.heads // 8))
        self.conv = None
        if self.taps:
            d = self.head_dim
            seg = lambda n, c: (self.names.get(n + "_conv", n + ".conv"), c)
            self.conv = build_part("filter", PartSpec("short_conv", {
                "channels": (self.heads + 2 * self.kv_heads) * d, "taps": self.taps, "state_name": "conv_tail",
                "segments": [seg("q", self.heads * d), seg("k", self.kv_heads * d), seg("v", self.kv_heads * d)]}, self.prefix), runtime)

    def _name(self, key):
        return self.prefix + self.names.get(key, key)

    def kernel_needs(self):
        return {"attention_head_dims": [self.head_dim], "libraries": ["prep"] + (["seq"] if self.taps else [])}

    def tensor_decls(self):
        sizes = [("q", self.heads * self.dim)] + ([("k", self.kv_heads * self.dim), ("v", self.kv_heads * self.vdim)] if self.own_kv else [])
        decls = [TensorDecl(self._name(n), (rows, self.hidden)) for n, rows in sizes]
        decls.append(TensorDecl(self._name("o"), (self.hidden, self.heads * self.vdim)))
        if self.bias:
            decls += [TensorDecl(self._name(n + ".b"), (rows,), role="vector", init="small") for n, rows in sizes]
        if self.out_bias:
            decls.append(TensorDecl(self._name("o.b"), (self.hidden,), role="vector", init="small"))
        if self.gate is not None:
            decls.append(TensorDecl(self._name("g"), (self.heads * self.vdim if self.gate == "element" else self.heads, self.hidden)))
        if self.taps:
            decls += [TensorDecl(self._name(n + ".conv"), (rows, self.taps)) for n, rows in sizes]
        if self.qk_norm_eps is not None:
            decls += [TensorDecl(self._name(n + ".norm"), (rows,), role="vector", init="norm") for n, rows in sizes if n != "v"]
        if self.sink:
            decls.append(TensorDecl(self._name("sink"), (self.heads,), role="vector", init="normal"))
        return decls

    def load(self, tensors):
        d = self.head_dim
        shapes = [("q", self.heads, self.dim)] + ([("k", self.kv_heads, self.dim), ("v", self.kv_heads, self.vdim)] if self.own_kv else [])
        rows = [_pad_heads(tensors[self._name(n)], h, size, d) for n, h, size in shapes]
        # the gate's projection rides along as more rows of the same product: its float sums are the gate
        if self.gate == "element":
            rows.append(_pad_heads(tensors[self._name("g")], self.heads, self.vdim, d))
        elif self.gate == "head":
            rows.append(_pad_heads(tensors[self._name("g")], 1, self.heads, self.gate_cols))
        self.w_in = torch.cat(rows, dim=0).contiguous()
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
        self.b_o = tensors[self._name("o.b")].float().contiguous() if self.out_bias else None
        self.sinks = tensors[self._name("sink")].float().contiguous() if self.sink else None
        if self.conv is not None:
            # the filters of the padded channels are zero, like the projection's padded rows
            padded = {self._name(n + ".conv"): _pad_heads(tensors[self._name(n + ".conv")], h, size, d) for n, h, size in shapes}
            self.conv.load({self.prefix + name: padded[self.prefix + name] for name, _ in self.conv.spec.params["segments"]})

    def cache_need(self):
        pages = CacheNeed(kv_heads=self.kv_heads, head_dim=self.head_dim, window=self.window, keep_first=self.keep_first)
        return pages if self.conv is None else CacheNeed.merged([("", pages), ("", self.conv.cache_need())])

    def output_weight(self):
        return self.w_o

    def mix_into(self, h, ctx, cache, out, scale: float = 1.0):
        if cache.writes != self.own_kv:
            raise ValueError("an attention without key/value tensors must read another execution's cache, and one with them its own")
        k = self.rt.kernels
        t, d = h.shape[0], self.head_dim
        n_qkv = (self.heads + 2 * self.cached_heads) * d
        sums = torch.empty((t, n_qkv + self.gate_cols), dtype=torch.float32, device=h.device)
        k.linear(h, self.w_in, sums)
        table = ctx.block_tables[cache.group]
        if self.conv is not None:
            proj = self.rt.empty_act((t, n_qkv))
            k.bias_round(sums[:, :n_qkv], self.b_in, proj)
            q = self.conv.forward(proj, ctx, cache)                        # [T, (H + 2 G) * D]: queries, then keys and values
            k.kv_norm_cache_write(q, ctx.positions, ctx.token_row, self.heads, self.kv_heads, d, 0, 0.0, cache.k, cache.v, table, cache.page_size)
        else:
            q = self.rt.empty_act((t, self.heads * d))
            per_head = self.head_norm_eps is not None
            eps = self.head_norm_eps if per_head else (self.qk_norm_eps if self.qk_norm_eps is not None else 0.0)
            k.qk_prepare(sums, self.b_in, ctx.positions, ctx.token_row, self.heads, self.cached_heads, d, self.dim, self.q_norm, self.k_norm,
                         eps, self.position.inv_freq, self.position.rotary_dim, q, cache.k, cache.v, table, cache.page_size,
                         **({"head_norm": True} if per_head else {}))
        direct = self.gate is None and scale == 1.0 and out.is_contiguous()
        attn = out if direct else self.rt.empty_act((t, self.heads * d))
        k.attention(q, cache.k, cache.v, table, ctx.cu_q, ctx.kv_len, ctx.token_row, ctx.positions, self.heads, self.kv_heads, d,
                    cache.page_size, self.scale, self.window or 0, attn, ctx.shape, sinks=self.sinks,
                    **({"keep_first": self.keep_first} if self.keep_first else {}))
        if not direct:
            gate = None if self.gate is None else sums[:, n_qkv: n_qkv + (self.heads if self.gate == "head" else self.gate_cols)]
            k.sigmoid_gate(attn, gate, out, scale)

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
