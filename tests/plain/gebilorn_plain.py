"""The Gebilorn decoder, whole sequences at a time, in plain torch on the CPU: one function per mechanism.

A slow restatement of the design's equations that shares no code with the engine; the tests compare the engine
with it. Every function takes one sequence ([T, ...] tensors, position 0 first) and works in the dtype of its
inputs (the tests use float64). Notation: T tokens, W width, H heads, G key/value heads.

The design: x_t = embed[tok_t] * s + bigram[(tok_(t-1) * a + tok_t * b) mod B] (row B for t = 0). A layer has one norm,
h = n(x), and both of its sub-layers read it: x += mixer(h) + ff(h); n(x) = x / rms(x) * (1 + w). Three mixers:
"attention" (grouped queries, partial rotation in the half layout with per-band scaled frequencies, queries and keys
divided by their own root mean square per head after the rotation, a window that also keeps the first tokens, a sink in
the softmax's denominator, an element-wise sigmoid gate on the heads' outputs), "parallel" (left: biased projections
through short causal convolutions, a plain window, a sink, one sigmoid gate per head; right: a matrix state per head
that decays per key channel, S <- diag(a_t) S + k_t v_t^T, read out after the update, normalised per head and gated by
silu; the two summed with fixed scales) and "latent_attention" (queries through a normalised low-rank step, keys and
values read out of one normalised low-rank vector per token plus one rotated key part that all heads share). The
feed-forward is dense and gated with the tanh form of gelu, or a mixture of silu-gated experts (softmax router, the
chosen scores times a constant as weights, a shared expert behind a sigmoid gate of one number per token), or absent.
Final norm, the embedding table as head, logits capped by c * tanh(l / c).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


# ---- small pieces -------------------------------------------------------------------------------------------
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, weight, eps):
    """RMS norm whose stored weight is the distance from one."""
    return unit_rms(x, eps) * (1.0 + weight)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def frequencies(rot: dict) -> List[float]:
    """One frequency per rotated pair: base^(-2i/dims), changed band by band if the file names a scaling: long waves
    are slowed by ``factor``, short ones stay, those between are blended."""
    dims = rot["dims"]
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = rot["base"] ** (-2.0 * i / dims)
        if sc:
            wave = 2.0 * math.pi / f
            if wave > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            elif wave >= sc["original"] / sc["high"]:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return out


def rotate(x, rot: Optional[dict]):
    """x [T, heads, D]: element i < dims/2 of a head pairs with element i + dims/2; the pair at position p turns by
    p * f_i. Elements from ``dims`` on pass unchanged."""
    if not rot or not rot.get("dims"):
        return x
    t, half = x.shape[0], rot["dims"] // 2
    out = x.clone()
    pos = torch.arange(t, dtype=x.dtype)
    for i, f in enumerate(frequencies(rot)):
        c, s = torch.cos(pos * f)[:, None], torch.sin(pos * f)[:, None]
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def visible(i: int, j: int, size: Optional[int], keep_first: int) -> bool:
    """May position i read position j? Not the future; inside the window, or one of the first tokens."""
    if j > i:
        return False
    return size is None or i - j < size or j < keep_first


def softmax_attention(q, k, v, scale, size, keep_first, sink):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]. ``sink`` [H] or None: exp(sink_h) joins the denominator."""
    t, heads, g = q.shape[0], q.shape[1], k.shape[1]
    allowed = torch.tensor([[visible(i, j, size, keep_first) for j in range(t)] for i in range(t)])
    out = torch.zeros(t, heads, v.shape[-1], dtype=q.dtype)
    for n in range(heads):
        kn, vn = k[:, n // (heads // g)], v[:, n // (heads // g)]
        s = ((q[:, n] @ kn.T) * scale).masked_fill(~allowed, -math.inf)
        top = s.max(-1, keepdim=True).values
        if sink is not None:
            top = torch.maximum(top, sink[n])
        e = torch.exp(s - top)
        den = e.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[n] - top)
        out[:, n] = (e / den) @ vn
    return out


def short_conv(u, filt):
    """u [T, C], filt [C, taps]: y_t = sum_j filt[:, j] * u_(t - taps + 1 + j), zeros before the start."""
    t, taps = u.shape[0], filt.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=u.dtype), u], 0)
    return sum(padded[j: j + t] * filt[:, j] for j in range(taps))


# ---- mixers ---------------------------------------------------------------------------------------------------
def attention_mixer(h, w, p, m, eps):
    heads, g, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    t = h.shape[0]
    q = rotate((h @ w[p + "q"].T).view(t, heads, dim), m.get("rot"))
    k = rotate((h @ w[p + "k"].T).view(t, g, dim), m.get("rot"))
    v = (h @ w[p + "v"].T).view(t, g, vdim)
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    mask = m.get("mask") or {}
    o = softmax_attention(q, k, v, m["scale"], mask.get("size"), mask.get("keep_first") or 0, w[p + "sink"])
    o = o.reshape(t, heads * vdim) * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def conv_window_attention(h, w, p, m):
    """The left side of a parallel pair."""
    heads, g, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    t = h.shape[0]
    proj = lambda n: short_conv(h @ w[p + n].T + w[p + n + ".b"], w[p + n + ".conv"])
    q, k, v = proj("q").view(t, heads, dim), proj("k").view(t, g, dim), proj("v").view(t, g, vdim)
    o = softmax_attention(q, k, v, m["scale"], m["mask"]["size"], 0, w[p + "sink"])
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(t, heads * vdim) @ w[p + "o"].T


def decaying_state_mixer(h, w, p, m, eps):
    """The right side of a parallel pair: S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head."""
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    t = h.shape[0]
    q = (h @ w[p + "q"].T).view(t, heads, dim) * dim ** -0.5
    k = (h @ w[p + "k"].T).view(t, heads, dim)
    v = (h @ w[p + "v"].T).view(t, heads, vdim)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    a = (torch.sigmoid(z) ** (1.0 / m["tau"])).view(t, heads, dim)
    out = torch.zeros(t, heads, vdim, dtype=h.dtype)
    for n in range(heads):
        S = torch.zeros(dim, vdim, dtype=h.dtype)
        for i in range(t):
            S = a[i, n][:, None] * S + torch.outer(k[i, n], v[i, n])
            out[i, n] = S.T @ q[i, n]
    y = (unit_rms(out, eps) * w[p + "norm"]).reshape(t, heads * vdim) * F.silu(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    return (m["left_scale"] * conv_window_attention(h, w, p + "left.", m["left"])
            + m["right_scale"] * decaying_state_mixer(h, w, p + "right.", m["right"], eps))


def latent_mixer(h, w, p, m, eps):
    heads, dim, rd, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    t = h.shape[0]
    rot = dict(m["rot"], dims=m["rot"].get("dims", rd))
    cq = unit_rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).view(t, heads, dim + rd)
    q_plain, q_rot = q[..., :dim], rotate(q[..., dim:], rot)
    down = h @ w[p + "dkv"].T
    c = unit_rms(down[:, :rank], eps) * w[p + "dkv.norm"]
    k_rot = rotate(down[:, rank:].view(t, 1, rd), rot)[:, 0]
    k_plain = (c @ w[p + "uk"].T).view(t, heads, dim)
    v = (c @ w[p + "uv"].T).view(t, heads, vdim)
    out = torch.zeros(t, heads, vdim, dtype=h.dtype)
    causal = torch.tril(torch.ones(t, t, dtype=torch.bool))
    for n in range(heads):
        s = (q_plain[:, n] @ k_plain[:, n].T + q_rot[:, n] @ k_rot.T) * m["scale"]
        out[:, n] = torch.softmax(s.masked_fill(~causal, -math.inf), -1) @ v[:, n]
    return out.reshape(t, heads * vdim) @ w[p + "o"].T


# ---- feed-forwards --------------------------------------------------------------------------------------------
def gated_ff(h, w, p, act):
    return (act(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def chosen_experts(h, w, p, f):
    """[T, top] indices of the experts with the largest scores (lowest index first on ties) and their weights."""
    s = torch.softmax(h @ w[p + "router"].T, -1)
    top = f["router"]["top"]
    idx = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
    return idx, torch.gather(s, 1, idx) * (f["router"].get("scale") or 1.0)


def expert_ff(h, w, p, f):
    idx, wt = chosen_experts(h, w, p, f)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for i in range(h.shape[0]):
        for e, c in zip(idx[i].tolist(), wt[i]):
            out[i] += c * gated_ff(h[i: i + 1], w, f"{p}e{e}.", F.silu)[0]
    if f.get("shared") is not None:
        out = out + gated_ff(h, w, p + "shared.", F.silu) * torch.sigmoid(h @ w[p + "shared.sg"].T)
    return out


def feed_forward(h, w, p, f):
    if f is None:
        return torch.zeros_like(h)
    return gated_ff(h, w, p, gelu_tanh) if f["kind"] == "dense" else expert_ff(h, w, p, f)


# ---- the model ------------------------------------------------------------------------------------------------
def embed(tokens, w, cfg):
    x = w["embed"][tokens] * (cfg.get("embedding") or {}).get("scale", 1.0)
    b = (cfg.get("embedding") or {}).get("bigram")
    if b:
        rows = [b["buckets"]] + [(tokens[i - 1] * b["mul_prev"] + tokens[i] * b["mul_cur"]) % b["buckets"] for i in range(1, len(tokens))]
        x = x + w["bigram"][torch.tensor(rows)]
    return x


def mixer(h, w, p, layer, eps):
    kind = layer["type"]
    if kind == "attention":
        return attention_mixer(h, w, p, layer["mixer"], eps)
    if kind == "parallel":
        return parallel_mixer(h, w, p, layer["mixer"], eps)
    return latent_mixer(h, w, p, layer["mixer"], eps)


def forward(tokens, w: Dict[str, torch.Tensor], cfg: dict, streams: Optional[list] = None):
    """Logits [T, vocab] of one sequence. ``streams``, if given, receives the residual stream after every layer."""
    tokens = [int(t) for t in tokens]
    eps = cfg["norm"]["eps"]
    x = embed(tokens, w, cfg)
    for i, layer in enumerate(cfg["layers"]):
        h = offset_norm(x, w[f"l{i}.norm1"], eps)
        x = x + (mixer(h, w, f"l{i}.mix.", layer, eps) + feed_forward(h, w, f"l{i}.mlp.", layer.get("mlp")))
        if streams is not None:
            streams.append(x.clone())
    logits = offset_norm(x, w["final.norm"], eps) @ w["embed"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits


# ---- tensor names and shapes ------------------------------------------------------------------------------------
def tensor_shapes(cfg: dict, decay_rank: int = 8) -> Dict[str, tuple]:
    """Every tensor of a model of this configuration; ``decay_rank`` is the width of the decay's two-step projection."""
    wd = cfg["width"]
    s: Dict[str, tuple] = {"embed": (cfg["vocab"], wd), "final.norm": (wd,)}
    b = (cfg.get("embedding") or {}).get("bigram")
    if b:
        s["bigram"] = (b["buckets"] + 1, wd)

    def gated(p, ff):
        s[p + "gate"], s[p + "up"], s[p + "down"] = (ff, wd), (ff, wd), (wd, ff)

    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        s[f"l{i}.norm1"] = (wd,)
        if layer["type"] == "attention":
            s[p + "q"], s[p + "k"], s[p + "v"] = (m["heads"] * m["dim"], wd), (m["kv_heads"] * m["dim"], wd), (m["kv_heads"] * m["vdim"], wd)
            s[p + "sink"], s[p + "g"], s[p + "o"] = (m["heads"],), (m["heads"] * m["vdim"], wd), (wd, m["heads"] * m["vdim"])
        elif layer["type"] == "parallel":
            l, r = m["left"], m["right"]
            for n, rows in (("q", l["heads"] * l["dim"]), ("k", l["kv_heads"] * l["dim"]), ("v", l["kv_heads"] * l["vdim"])):
                s[p + "left." + n], s[p + "left." + n + ".b"], s[p + "left." + n + ".conv"] = (rows, wd), (rows,), (rows, l["conv"])
            s[p + "left.sink"], s[p + "left.g"], s[p + "left.o"] = (l["heads"],), (l["heads"], wd), (wd, l["heads"] * l["vdim"])
            hk, hv = r["heads"] * r["dim"], r["heads"] * r["vdim"]
            s[p + "right.q"], s[p + "right.k"], s[p + "right.v"], s[p + "right.g"] = (hk, wd), (hk, wd), (hv, wd), (hv, wd)
            s[p + "right.o"], s[p + "right.norm"] = (wd, hv), (r["vdim"],)
            s[p + "right.a1"], s[p + "right.a2"], s[p + "right.a2.b"] = (decay_rank, wd), (hk, decay_rank), (hk,)
        else:
            s[p + "dq"], s[p + "dq.norm"], s[p + "uq"] = (m["q_rank"], wd), (m["q_rank"],), (m["heads"] * (m["dim"] + m["rot_dim"]), m["q_rank"])
            s[p + "dkv"], s[p + "dkv.norm"] = (m["kv_rank"] + m["rot_dim"], wd), (m["kv_rank"],)
            s[p + "uk"], s[p + "uv"] = (m["heads"] * m["dim"], m["kv_rank"]), (m["heads"] * m["vdim"], m["kv_rank"])
            s[p + "o"] = (wd, m["heads"] * m["vdim"])
        f = layer.get("mlp")
        if f is None:
            continue
        p = f"l{i}.mlp."
        if f["kind"] == "dense":
            gated(p, f["ff"])
        else:
            s[p + "router"] = (f["router"]["experts"], wd)
            for e in range(f["router"]["experts"]):
                gated(f"{p}e{e}.", f["expert"]["ff"])
            if f.get("shared") is not None:
                gated(p + "shared.", f["shared"]["ff"])
                s[p + "shared.sg"] = (1, wd)
    return s
