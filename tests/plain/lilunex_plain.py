"""The Lilunex decoder, whole sequences at a time, in plain torch on the CPU: one function per mechanism.

A slow restatement of the design's equations that shares no code with the engine; the tests compare the engine
with it. Every function takes one sequence ([T, ...] tensors, position 0 first) and works in the dtype of its
inputs (the tests use float64 or float32). Notation: T tokens, W width, H heads, G key/value heads.

The design: x = embed[token] * s. A layer is x += n1b(mixer(n1(x))); x += n2b(ff(n2(x))), every n a "dynamic tanh",
tanh(alpha x) * w + b with a scalar alpha. Three mixers: "wkv" (token-shifted inputs, a matrix state per head with a
decay per key channel that depends on the token, and a bonus for the current token), "attention" (biased projections,
queries and keys normalised over the whole projection, partial rotation with linearly scaled frequencies, a window
that also keeps the first tokens, a sink in the softmax's denominator, optionally another layer's keys and values)
and "delta" (gated delta rule with one decay per head). Feed-forwards: dense with relu squared, or a mixture of gated
experts with a softmax router, a choice bias, identity experts and a gated shared expert. Final norm, untied head.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch
import torch.nn.functional as F


# ---- small pieces -------------------------------------------------------------------------------------------
def dyn_tanh(x, w, name):
    """tanh(alpha x) * weight + bias; alpha is a scalar."""
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rotate_half_layout(x, base: float, dims: int, factor: float):
    """x [T, heads, D]: element i < dims/2 of a head pairs with element i + dims/2; the pair at position p turns by the
    angle p * base^(-2i/dims) / factor. Elements from ``dims`` on pass unchanged."""
    t = x.shape[0]
    half = dims // 2
    out = x.clone()
    pos = torch.arange(t, dtype=x.dtype)
    for i in range(half):
        f = base ** (-2.0 * i / dims) / factor
        c, s = torch.cos(pos * f)[:, None], torch.sin(pos * f)[:, None]
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def visible(i: int, j: int, size: int, keep_first: int) -> bool:
    """May position i read position j? Causal, inside the window, or one of the first tokens."""
    return j <= i and (i - j < size or j < keep_first)


# ---- mixers ---------------------------------------------------------------------------------------------------
def wkv_mixer(h, w, p, m, eps):
    """Token-shifted projections, then per head o_t = (S + diag(u) k_t v_t^T)^T r_t and S <- diag(d_t) S + k_t v_t^T."""
    heads, dim = m["heads"], m["dim"]
    t = h.shape[0]
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)
    mix = {s: h + (prev - h) * w[p + "mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ w[p + "r"].T).view(t, heads, dim)
    k = (mix["k"] @ w[p + "k"].T).view(t, heads, dim)
    v = (mix["v"] @ w[p + "v"].T).view(t, heads, dim)
    gate = F.silu(mix["g"] @ w[p + "g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix["w"] @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(t, heads, dim)
    u = w[p + "u"]
    out = torch.zeros(t, heads, dim, dtype=h.dtype)
    for n in range(heads):
        S = torch.zeros(dim, dim, dtype=h.dtype)
        for i in range(t):
            kv = torch.outer(k[i, n], v[i, n])
            out[i, n] = (S + u[n][:, None] * kv).T @ r[i, n]
            S = decay[i, n][:, None] * S + kv
    y = unit_rms(out, eps).reshape(t, heads * dim) * w[p + "norm"] * gate
    return y @ w[p + "o"].T


def _rot_factor(m) -> float:
    scaling = (m.get("rot") or {}).get("scaling")
    return float(scaling["factor"]) if scaling else 1.0


def _rotated(x, m):
    rot = m.get("rot")
    return rotate_half_layout(x, rot["base"], rot["dims"], _rot_factor(m)) if rot else x


def attention_keys_values(h, w, p, m, eps):
    """What an attention layer caches: keys after norm and rotation [T, G, dim], values [T, G, vdim]."""
    g, dim, vdim = m["kv_heads"], m["dim"], m["vdim"]
    t = h.shape[0]
    k = h @ w[p + "k"].T + w[p + "k.b"]
    v = h @ w[p + "v"].T + w[p + "v.b"]
    k = unit_rms(k, eps) * w[p + "k.norm"]
    k = _rotated(k.view(t, g, dim), m)
    return k, v.view(t, g, vdim)


def attention_mixer(h, w, p, m, eps, k, v):
    """Grouped-query attention over given keys and values, with its own queries, mask and sink."""
    heads, g, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    t = h.shape[0]
    q = h @ w[p + "q"].T + w[p + "q.b"]
    q = unit_rms(q, eps) * w[p + "q.norm"]
    q = _rotated(q.view(t, heads, dim), m)
    mask = m.get("mask")
    size, keep = (mask["size"], mask.get("keep_first") or 0) if mask else (t + 1, 0)
    allowed = torch.tensor([[visible(i, j, size, keep) for j in range(t)] for i in range(t)])
    out = torch.zeros(t, heads, vdim, dtype=h.dtype)
    for n in range(heads):
        kn, vn = k[:, n // (heads // g)], v[:, n // (heads // g)]
        s = (q[:, n] @ kn.T) * m["scale"]
        s = s.masked_fill(~allowed, -math.inf)
        sink = w[p + "sink"][n]
        top = torch.maximum(s.max(-1, keepdim=True).values, sink)
        e = torch.exp(s - top)
        out[:, n] = (e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))) @ vn
    return out.reshape(t, heads * vdim) @ w[p + "o"].T + w[p + "o.b"]


def short_conv_silu(x, filt):
    """x [T, C], filt [C, taps]: out[t] = silu(sum_j filt[:, j] x[t - taps + 1 + j]), zeros before the start."""
    t, taps = x.shape[0], filt.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=x.dtype), x], 0)
    out = torch.zeros_like(x)
    for j in range(taps):
        out = out + padded[j: j + t] * filt[:, j]
    return F.silu(out)


def delta_mixer(h, w, p, m, eps):
    """Gated delta rule: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    heads, g, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    t = h.shape[0]
    q = short_conv_silu(h @ w[p + "q"].T, w[p + "q.conv"]).view(t, g, dim)
    k = short_conv_silu(h @ w[p + "k"].T, w[p + "k.conv"]).view(t, g, dim)
    v = short_conv_silu(h @ w[p + "v"].T, w[p + "v.conv"]).view(t, heads, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * F.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    out = torch.zeros(t, heads, vdim, dtype=h.dtype)
    for n in range(heads):
        S = torch.zeros(dim, vdim, dtype=h.dtype)
        c = n // (heads // g)
        for i in range(t):
            S = decay[i, n] * S
            u = beta[i, n] * (v[i, n] - S.T @ k[i, c])
            S = S + torch.outer(k[i, c], u)
            out[i, n] = S.T @ q[i, c]
    gate = F.silu(h @ w[p + "g"].T).view(t, heads, vdim)
    y = unit_rms(out, eps) * w[p + "norm"] * gate
    return y.reshape(t, heads * vdim) @ w[p + "o"].T


# ---- feed-forwards --------------------------------------------------------------------------------------------
def dense_ff(h, w, p):
    return torch.relu(h @ w[p + "up"].T) ** 2 @ w[p + "down"].T


def gated_expert(h, w, p):
    return (F.silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def router_choice(h, w, p, f):
    """(chosen indices [T, top], weights [T, top]): softmax over experts and identity experts; the choice adds the
    correction, the weights do not; weights are divided by their sum."""
    s = torch.softmax(h @ w[p + "router"].T, -1)
    chosen = torch.topk(s + w[p + "correction"], f["router"]["top"], dim=-1).indices
    picked = torch.gather(s, 1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + 1e-20)


def moe_ff(h, w, p, f):
    n_real = f["router"]["experts"]
    chosen, weights = router_choice(h, w, p, f)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t].tolist(), weights[t]):
            out[t] += wt * (h[t] if e >= n_real else gated_expert(h[t: t + 1], w, f"{p}e{e}.")[0])
    if f.get("shared") is not None:
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * gated_expert(h, w, p + "shared.")
    return out


# ---- the model --------------------------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one sequence. ``layers_out``: a list that receives the residual stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * (cfg["embedding"]["scale"] if cfg.get("embedding") else 1.0)
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = dyn_tanh(x, w, p + "norm1")
        if layer["type"] == "wkv":
            a = wkv_mixer(h, w, p + "mix.", m, eps)
        elif layer["type"] == "delta":
            a = delta_mixer(h, w, p + "mix.", m, eps)
        else:
            if m.get("kv_from") is None:
                kept[i] = attention_keys_values(h, w, p + "mix.", m, eps)
            a = attention_mixer(h, w, p + "mix.", m, eps, *kept[i if m.get("kv_from") is None else m["kv_from"]])
        x = x + dyn_tanh(a, w, p + "norm1b")
        f = layer["mlp"]
        if f is not None:
            h = dyn_tanh(x, w, p + "norm2")
            d = dense_ff(h, w, p + "mlp.") if f["kind"] == "dense" else moe_ff(h, w, p + "mlp.", f)
            x = x + dyn_tanh(d, w, p + "norm2b")
        if layers_out is not None:
            layers_out.append(x.clone())
    return dyn_tanh(x, w, "final.norm") @ w["head"].T


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """Names and shapes of a model's tensors (``rank`` of the decay's two-step projection: cfg layers' mixer["rank"])."""
    width, out = cfg["width"], {}

    def norm(name):
        out[name], out[name + ".b"], out[name + ".alpha"] = (width,), (width,), ()

    out["embed"] = (cfg["vocab"], width)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        norm(p + "norm1"); norm(p + "norm1b")
        q = p + "mix."
        if layer["type"] == "wkv":
            hd = m["heads"] * m["dim"]
            for s in "rkvgw":
                out[q + "mu." + s] = (width,)
            for s in "rkvg":
                out[q + s] = (hd, width)
            rank = m.get("rank", 8)
            out[q + "w1"], out[q + "w2"], out[q + "w0"] = (rank, width), (hd, rank), (hd,)
            out[q + "u"], out[q + "norm"], out[q + "o"] = (m["heads"], m["dim"]), (hd,), (width, hd)
        elif layer["type"] == "delta":
            qk, hv = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
            for s, n in (("q", qk), ("k", qk), ("v", hv)):
                out[q + s], out[q + s + ".conv"] = (n, width), (n, m["conv"])
            out[q + "b"], out[q + "a"] = (m["heads"], width), (m["heads"], width)
            out[q + "A_log"], out[q + "dt_bias"], out[q + "norm"] = (m["heads"],), (m["heads"],), (m["vdim"],)
            out[q + "g"], out[q + "o"] = (hv, width), (width, hv)
        else:
            hq, hk, hv = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
            out[q + "q"], out[q + "q.b"], out[q + "q.norm"] = (hq, width), (hq,), (hq,)
            if m.get("kv_from") is None:
                out[q + "k"], out[q + "k.b"], out[q + "k.norm"] = (hk, width), (hk,), (hk,)
                out[q + "v"], out[q + "v.b"] = (hv, width), (hv,)
            out[q + "sink"] = (m["heads"],)
            out[q + "o"], out[q + "o.b"] = (width, m["heads"] * m["vdim"]), (width,)
        f = layer["mlp"]
        if f is None:
            continue
        norm(p + "norm2"); norm(p + "norm2b")
        q = p + "mlp."
        if f["kind"] == "dense":
            out[q + "up"], out[q + "down"] = (f["ff"], width), (width, f["ff"])
        else:
            r = f["router"]
            for e in range(r["experts"]):
                out[f"{q}e{e}.gate"], out[f"{q}e{e}.up"], out[f"{q}e{e}.down"] = (f["expert"]["ff"], width), (f["expert"]["ff"], width), (width, f["expert"]["ff"])
            n = r["experts"] + (r.get("identity") or 0)
            out[q + "router"], out[q + "correction"] = (n, width), (n,)
            if f.get("shared") is not None:
                sf = f["shared"]["ff"]
                out[q + "shared.gate"], out[q + "shared.up"], out[q + "shared.down"] = (sf, width), (sf, width), (width, sf)
                out[q + "shared.sg"] = (1, width)
    norm("final.norm")
    out["head"] = (cfg["vocab"], width)
    return out
