"""Mixers that carry a matrix state per head from token to token instead of a cache of keys.

All of them keep S [dk, dv] per (request, head) in float and differ in how a token changes it:

  "lightning"    S <- decay_h S + k v^T,  o = S^T q          q, k, v = silu of their projections; decay_h fixed per head
  "mamba2"       S <- exp(-exp(A_h) dt) S + dt B x^T,  y = S^T C + D_h x      dt = softplus(dt' + bias_h); x, B, C pass a
                 short convolution and silu first; heads share B and C in groups
  "gated_delta"  S <- g . S (a decay per row of S, or one per head);  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
                 q, k, v pass a short convolution and silu, q and k become unit vectors, q times dk^-1/2
  "wkv"          o = (S + diag(u_h) k v^T)^T r;  S <- diag(d) S + k v^T      r, k, v, the gate and the decay each read
                 their own blend of the token's input with the one before; d = exp(-exp(w0 + W2 tanh(W1 x_w))) per key
                 channel; the bonus u_h counts for the current token only, and the read-out comes before the update
  "gated_linear_attention"  S <- diag(a) S + k v^T,  o = S^T q      q times dk^-1/2; a = sigmoid(W_a2 (W_a1 h) + b)^(1/tau) per key
                 channel, formed in float as exp(log_sigmoid(z) / tau); the read-out comes after the update

The read-out goes through a root-mean-square norm with a gate (parts/gated_norm.py) and an output projection.
One kernel walks the tokens of every request of the step in order (csrc/sequence_ops.cu), so a prompt cut into
portions, or decoded token by token, runs the same arithmetic in the same order as the whole prompt at once.
"""
from __future__ import annotations

import math

import torch

from ..config.spec import PartSpec
from .base import CacheNeed, Mixer, TensorDecl, build_part, register_part


class RecurrentMixer(Mixer):
    """What the three share: input projections fused into one product, a float read-out, norm and gate, output projection."""

    def _common(self, p):
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.eps = float(p["eps"])
        self.names = dict(p.get("names", {}))

    def _name(self, key):
        return self.prefix + self.names.get(key, key)

    def output_weight(self):
        return self.w_o

    def forward(self, h, ctx, cache):
        mixed = self.rt.empty_act((h.shape[0], self.mixed_size))
        self.mix_into(h, ctx, cache, mixed)
        out = self.rt.empty_act((h.shape[0], self.hidden))
        self.rt.kernels.linear(mixed, self.w_o, out)
        return out

    def _readout(self, t):
        return torch.empty((t, self.mixed_size), dtype=torch.float32, device=self.rt.device)


@register_part("mixer", "lightning")
class LightningMixer(RecurrentMixer):
    """params: hidden, heads, dim, vdim, decay (one per head), eps."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self._common(p)
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.decay_values = [float(d) for d in p["decay"]]
        if len(self.decay_values) != self.heads:
            raise ValueError(f"{len(self.decay_values)} decays for {self.heads} heads")
        self.mixed_size = self.heads * self.vdim
        self.norm = build_part("norm", PartSpec("gated_group_rms", {"channels": self.mixed_size, "groups": 1, "eps": self.eps,
                                                                    "weight_name": self.names.get("norm", "norm"), "gate": "sigmoid"},
                                                self.prefix), runtime)
        self.decay = None

    def tensor_decls(self):
        hk, hv = self.heads * self.dim, self.heads * self.vdim
        return [TensorDecl(self._name("q"), (hk, self.hidden)), TensorDecl(self._name("k"), (hk, self.hidden)),
                TensorDecl(self._name("v"), (hv, self.hidden)), TensorDecl(self._name("g"), (hv, self.hidden)),
                TensorDecl(self._name("o"), (self.hidden, hv))] + self.norm.tensor_decls()

    def load(self, tensors):
        self.w_in = torch.cat([tensors[self._name(n)] for n in ("q", "k", "v", "g")], dim=0).contiguous()
        self.w_o = tensors[self._name("o")].contiguous()
        self.norm.load(tensors)
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.w_o.device)

    def cache_need(self):
        return CacheNeed(states=(("state", (self.heads, self.dim, self.vdim)),))

    def mix_into(self, h, ctx, cache, out, scale: float = 1.0):
        k = self.rt.kernels
        t, hk, hv = h.shape[0], self.heads * self.dim, self.heads * self.vdim
        proj = self.rt.empty_act((t, 2 * hk + 2 * hv))
        k.linear(h, self.w_in, proj)
        y = self._readout(t)
        k.linear_recurrence("decay", proj[:, :hk], proj[:, hk: 2 * hk], proj[:, 2 * hk: 2 * hk + hv], cache.states["state"], ctx, y,
                            self.heads, self.heads, self.dim, self.vdim, decay=self.decay)
        self.norm.forward(y, proj[:, 2 * hk + hv:], out, scale)


@register_part("mixer", "mamba2")
class Mamba2Mixer(RecurrentMixer):
    """params: hidden, heads, vdim, state, groups, norm_groups, taps, eps."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self._common(p)
        self.vdim, self.n, self.groups = int(p["vdim"]), int(p["state"]), int(p["groups"])
        if self.heads % self.groups:
            raise ValueError(f"{self.heads} heads do not split into {self.groups} groups")
        self.inner = self.mixed_size = self.heads * self.vdim
        self.conv_channels = self.inner + 2 * self.groups * self.n
        self.conv = build_part("filter", PartSpec("short_conv", {
            "channels": self.conv_channels, "taps": int(p["taps"]), "weight_name": self.names.get("conv", "conv"),
            "bias_name": self.names.get("conv_bias", "conv.b"), "activation": "silu", "state_name": "conv_tail"}, self.prefix), runtime)
        self.norm = build_part("norm", PartSpec("gated_group_rms", {
            "channels": self.inner, "groups": int(p["norm_groups"]), "eps": self.eps, "weight_name": self.names.get("norm", "norm"),
            "gate": "silu", "gate_first": True}, self.prefix), runtime)

    def tensor_decls(self):
        vec = lambda n: TensorDecl(self._name(n), (self.heads,), role="vector", init="norm")
        return ([TensorDecl(self._name("in"), (2 * self.inner + 2 * self.groups * self.n + self.heads, self.hidden)),
                 TensorDecl(self._name("o"), (self.hidden, self.inner)), vec("dt_bias"), vec("A_log"), vec("D")]
                + self.conv.tensor_decls() + self.norm.tensor_decls())

    def load(self, tensors):
        self.w_in = tensors[self._name("in")].contiguous()
        self.w_o = tensors[self._name("o")].contiguous()
        self.dt_bias, self.a_log, self.d_skip = (tensors[self._name(n)].contiguous() for n in ("dt_bias", "A_log", "D"))
        self.conv.load(tensors)
        self.norm.load(tensors)

    def cache_need(self):
        return CacheNeed.merged([("", CacheNeed(states=(("state", (self.heads, self.n, self.vdim)),))), ("", self.conv.cache_need())])

    def mix_into(self, h, ctx, cache, out, scale: float = 1.0):
        k = self.rt.kernels
        t, inner, gn = h.shape[0], self.inner, self.groups * self.n
        proj = self.rt.empty_act((t, 2 * inner + 2 * gn + self.heads))
        k.linear(h, self.w_in, proj)
        xbc = self.conv.forward(proj[:, inner: 2 * inner + 2 * gn], ctx, cache)
        y = self._readout(t)
        k.linear_recurrence("ssm", xbc[:, inner + gn:], xbc[:, inner: inner + gn], xbc[:, :inner], cache.states["state"], ctx, y,
                            self.heads, self.groups, self.n, self.vdim, aux=proj[:, 2 * inner + 2 * gn:], a_log=self.a_log,
                            dt_bias=self.dt_bias, d_skip=self.d_skip)
        self.norm.forward(y, proj[:, :inner], out, scale)


@register_part("mixer", "gated_delta")
class GatedDeltaMixer(RecurrentMixer):
    """params: hidden, heads, kv_heads, dim, vdim, taps, eps, rank (width of the two-step projections of the decay rate
    and of the gate; None: whatever the weight file has); decay_per ("channel": a rate per row of S, dt_bias [heads * dim];
    "head": one rate per head, dt_bias [heads]); low_rank (True: rate and gate come through two-step projections a1/a2 and
    g1/g2; False: each is one projection of the layer's input, named "rate" and "gate"); gate ("sigmoid" | "silu")."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self._common(p)
        self.kv_heads, self.dim, self.vdim = int(p["kv_heads"]), int(p["dim"]), int(p["vdim"])
        if self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        self.rank = int(p["rank"]) if p.get("rank") else -1
        self.per_head = p.get("decay_per", "channel") == "head"
        if p.get("decay_per", "channel") not in ("channel", "head"):
            raise ValueError(f"gated_delta: decay_per {p['decay_per']!r} is not known (channel, head)")
        self.low_rank = bool(p.get("low_rank", True))
        self.rate_size = self.heads if self.per_head else self.heads * self.dim
        self.qk, self.mixed_size = self.kv_heads * self.dim, self.heads * self.vdim
        seg = lambda n, c: (self.names.get(n + "_conv", n + ".conv"), c)
        self.conv = build_part("filter", PartSpec("short_conv", {
            "channels": 2 * self.qk + self.mixed_size, "taps": int(p["taps"]), "activation": "silu", "state_name": "conv_tail",
            "segments": [seg("q", self.qk), seg("k", self.qk), seg("v", self.mixed_size)]}, self.prefix), runtime)
        self.norm = build_part("norm", PartSpec("gated_group_rms", {
            "channels": self.mixed_size, "groups": self.heads, "eps": self.eps, "weight_size": self.vdim,
            "weight_name": self.names.get("norm", "norm"), "gate": p.get("gate", "sigmoid")}, self.prefix), runtime)

    def kernel_needs(self):
        return {"libraries": ["seq"]}

    def tensor_decls(self):
        hid, r = self.hidden, self.rank
        if self.low_rank:
            two_step = [TensorDecl(self._name("a1"), (r, hid)), TensorDecl(self._name("a2"), (self.rate_size, r)),
                        TensorDecl(self._name("g1"), (r, hid)), TensorDecl(self._name("g2"), (self.mixed_size, r))]
        else:
            two_step = [TensorDecl(self._name("rate"), (self.rate_size, hid)), TensorDecl(self._name("gate"), (self.mixed_size, hid))]
        return ([TensorDecl(self._name("q"), (self.qk, hid)), TensorDecl(self._name("k"), (self.qk, hid)),
                 TensorDecl(self._name("v"), (self.mixed_size, hid)), TensorDecl(self._name("b"), (self.heads, hid))] + two_step
                + [TensorDecl(self._name("o"), (hid, self.mixed_size)),
                   TensorDecl(self._name("A_log"), (self.heads,), role="vector", init="norm"),
                   TensorDecl(self._name("dt_bias"), (self.rate_size,), role="vector", init="norm")]
                + self.conv.tensor_decls() + self.norm.tensor_decls())

    def load(self, tensors):
        t = lambda n: tensors[self._name(n)]
        if self.low_rank:
            if t("a1").shape[0] != t("a2").shape[1] or t("g1").shape[0] != t("g2").shape[1]:
                raise ValueError(f"{self.prefix}: the two steps of a low-rank projection do not fit each other")
            self.rank_a, self.rank_g = t("a1").shape[0], t("g1").shape[0]
            self.w_in = torch.cat([t(n) for n in ("q", "k", "v", "b", "a1", "g1")], dim=0).contiguous()
            self.w_a2, self.w_g2 = t("a2").contiguous(), t("g2").contiguous()
        else:
            self.w_in = torch.cat([t(n) for n in ("q", "k", "v", "b", "rate", "gate")], dim=0).contiguous()
        self.w_o = t("o").contiguous()
        self.a_log, self.dt_bias = t("A_log").contiguous(), t("dt_bias").contiguous()
        self.conv.load(tensors)
        self.norm.load(tensors)

    def cache_need(self):
        return CacheNeed.merged([("", CacheNeed(states=(("state", (self.heads, self.dim, self.vdim)),))), ("", self.conv.cache_need())])

    def mix_into(self, h, ctx, cache, out, scale: float = 1.0):
        k = self.rt.kernels
        t, qk, hv, hd = h.shape[0], self.qk, self.mixed_size, self.heads
        n_conv = 2 * qk + hv
        at = n_conv + hd
        if self.low_rank:
            proj = self.rt.empty_act((t, at + self.rank_a + self.rank_g))
            k.linear(h, self.w_in, proj)
            rate = self.rt.empty_act((t, self.rate_size))
            k.linear(proj[:, at: at + self.rank_a], self.w_a2, rate)
            gate = self.rt.empty_act((t, hv))
            k.linear(proj[:, at + self.rank_a:], self.w_g2, gate)
        else:
            proj = self.rt.empty_act((t, at + self.rate_size + hv))
            k.linear(h, self.w_in, proj)
            rate, gate = proj[:, at: at + self.rate_size], proj[:, at + self.rate_size:]
        qkv = self.conv.forward(proj[:, :n_conv], ctx, cache)
        y = self._readout(t)
        k.linear_recurrence("delta", qkv[:, :qk], qkv[:, qk: 2 * qk], qkv[:, 2 * qk:], cache.states["state"], ctx, y, hd, self.kv_heads,
                            self.dim, self.vdim, aux=proj[:, n_conv: n_conv + hd], rate=rate, a_log=self.a_log, dt_bias=self.dt_bias,
                            q_scale=1.0 / math.sqrt(self.dim), **({"rate_per_head": True} if self.per_head else {}))
        self.norm.forward(y, gate, out, scale)


@register_part("mixer", "wkv")
class WkvMixer(RecurrentMixer):
    """params: hidden, heads, dim, eps, rank (width of the decay's two-step projection; None: whatever the weight file has).
    Tensors: blend vectors "mu.r/k/v/g/w", projections "r", "k", "v", "g" [heads * dim, hidden], "w1" [rank, hidden], "w2"
    [heads * dim, rank], "w0" [heads * dim], bonus "u" [heads, dim], "norm" [heads * dim], "o"."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self._common(p)
        self.dim = int(p["dim"])
        self.rank = int(p["rank"]) if p.get("rank") else -1
        self.mixed_size = self.heads * self.dim
        self.shift = build_part("filter", PartSpec("token_shift", {
            "channels": self.hidden, "mixes": [self.names.get("mu." + s, "mu." + s) for s in "rkvgw"]}, self.prefix), runtime)
        self.norm = build_part("norm", PartSpec("gated_group_rms", {
            "channels": self.mixed_size, "groups": self.heads, "eps": self.eps, "weight_name": self.names.get("norm", "norm"),
            "gate": "silu"}, self.prefix), runtime)

    def kernel_needs(self):
        return {"libraries": ["seq"]}

    def tensor_decls(self):
        hid, n = self.hidden, self.mixed_size
        return ([TensorDecl(self._name(s), (n, hid)) for s in "rkvg"]
                + [TensorDecl(self._name("w1"), (self.rank, hid)), TensorDecl(self._name("w2"), (n, self.rank)),
                   TensorDecl(self._name("w0"), (n,), role="vector", init="norm"),
                   TensorDecl(self._name("u"), (self.heads, self.dim), role="vector", init="normal"),
                   TensorDecl(self._name("o"), (hid, n))]
                + self.shift.tensor_decls() + self.norm.tensor_decls())

    def load(self, tensors):
        t = lambda n: tensors[self._name(n)]
        if t("w1").shape[0] != t("w2").shape[1]:
            raise ValueError(f"{self.prefix}: the two steps of the decay's projection do not fit each other")
        self.w_rkvg = torch.stack([t(s) for s in "rkvg"]).contiguous()
        self.w1, self.w2, self.w_o = t("w1").contiguous(), t("w2").contiguous(), t("o").contiguous()
        self.w0, self.bonus = t("w0").float().contiguous(), t("u").float().reshape(-1).contiguous()
        self.shift.load(tensors)
        self.norm.load(tensors)

    def cache_need(self):
        return CacheNeed.merged([("", CacheNeed(states=(("state", (self.heads, self.dim, self.dim)),))), ("", self.shift.cache_need())])

    def mix_into(self, h, ctx, cache, out, scale: float = 1.0):
        k = self.rt.kernels
        t, n = h.shape[0], self.mixed_size
        blends = self.shift.forward(h, ctx, cache)                      # [5, T, hidden]: for r, k, v, the gate and the decay
        proj = self.rt.empty_act((t, 4, n))
        k.linear_batched(blends[:4].transpose(0, 1), self.w_rkvg, proj)
        low = self.rt.empty_act((t, self.w1.shape[0]))
        k.linear(blends[4], self.w1, low)
        k.activation(low, low, "tanh")
        rate = torch.empty((t, n), dtype=torch.float32, device=h.device)
        k.linear(low, self.w2, rate)
        y = self._readout(t)
        k.linear_recurrence("wkv", proj[:, 0], proj[:, 1], proj[:, 2], cache.states["state"], ctx, y, self.heads, self.heads, self.dim,
                            self.dim, rate=rate, dt_bias=self.w0, bonus=self.bonus)
        self.norm.forward(y, proj[:, 3], out, scale)


@register_part("mixer", "gated_linear_attention")
class GatedLinearAttention(RecurrentMixer):
    """params: hidden, heads, dim, vdim, tau, eps, rank (width of the decay's two-step projection; None: whatever the
    weight file has). Tensors: "q", "k" [heads * dim, hidden], "v", "g" [heads * vdim, hidden], "a1" [rank, hidden], "a2"
    [heads * dim, rank], "a2.b" [heads * dim], "norm" [vdim] (one weight for every head), "o". The read-out is divided by
    its root mean square per head, multiplied by the weight and by silu(W_g h)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self._common(p)
        self.dim, self.vdim, self.tau = int(p["dim"]), int(p["vdim"]), float(p["tau"])
        if not self.tau > 0:
            raise ValueError("gated_linear_attention: tau must be positive")
        self.rank = int(p["rank"]) if p.get("rank") else -1
        self.qk, self.mixed_size = self.heads * self.dim, self.heads * self.vdim
        self.norm = build_part("norm", PartSpec("gated_group_rms", {
            "channels": self.mixed_size, "groups": self.heads, "eps": self.eps, "weight_size": self.vdim,
            "weight_name": self.names.get("norm", "norm"), "gate": "silu"}, self.prefix), runtime)

    def kernel_needs(self):
        return {"libraries": ["seq"]}

    def tensor_decls(self):
        hid = self.hidden
        return ([TensorDecl(self._name("q"), (self.qk, hid)), TensorDecl(self._name("k"), (self.qk, hid)),
                 TensorDecl(self._name("v"), (self.mixed_size, hid)), TensorDecl(self._name("g"), (self.mixed_size, hid)),
                 TensorDecl(self._name("a1"), (self.rank, hid)), TensorDecl(self._name("a2"), (self.qk, self.rank)),
                 TensorDecl(self._name("a2.b"), (self.qk,), role="vector", init="small"),
                 TensorDecl(self._name("o"), (hid, self.mixed_size))] + self.norm.tensor_decls())

    def load(self, tensors):
        t = lambda n: tensors[self._name(n)]
        if t("a1").shape[0] != t("a2").shape[1]:
            raise ValueError(f"{self.prefix}: the two steps of the decay's projection do not fit each other")
        self.rank_a = t("a1").shape[0]
        # one product for q, k, v, the gate and the decay's first step (its rows padded to a multiple of 8 with zeros)
        pad = -self.rank_a % 8
        a1 = torch.cat([t("a1"), t("a1").new_zeros((pad, self.hidden))], 0) if pad else t("a1")
        self.w_in = torch.cat([t("q"), t("k"), t("v"), t("g"), a1], dim=0).contiguous()
        a2 = torch.cat([t("a2"), t("a2").new_zeros((self.qk, pad))], 1) if pad else t("a2")
        self.w_a2 = a2.contiguous()
        self.rank_p = self.rank_a + pad
        self.b_a2 = t("a2.b").float().contiguous()
        self.w_o = t("o").contiguous()
        self.norm.load(tensors)

    def cache_need(self):
        return CacheNeed(states=(("state", (self.heads, self.dim, self.vdim)),))

    def mix_into(self, h, ctx, cache, out, scale: float = 1.0):
        k = self.rt.kernels
        t, hk, hv = h.shape[0], self.qk, self.mixed_size
        proj = self.rt.empty_act((t, 2 * hk + 2 * hv + self.rank_p))
        k.linear(h, self.w_in, proj)
        rate = torch.empty((t, hk), dtype=torch.float32, device=h.device)     # float sums: what enters the recurrence is not rounded
        k.linear(proj[:, 2 * hk + 2 * hv:], self.w_a2, rate)
        y = self._readout(t)
        k.linear_recurrence("gla", proj[:, :hk], proj[:, hk: 2 * hk], proj[:, 2 * hk: 2 * hk + hv], cache.states["state"], ctx, y,
                            self.heads, self.heads, self.dim, self.vdim, rate=rate, dt_bias=self.b_a2,
                            q_scale=1.0 / math.sqrt(self.dim), rate_scale=1.0 / self.tau)
        self.norm.forward(y, proj[:, 2 * hk + hv: 2 * hk + 2 * hv], out, scale)
