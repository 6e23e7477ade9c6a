"""Shared by the Gebilorn tests: small configurations of their own, seeded weights, engines on either backend.

Two backends: "emu" runs the engine's own parts, cache manager and step function on the CPU over the torch stand-ins of
tests/emu_kernels.py (no GPU needed, float32); "cuda" runs the real kernels. The oracle is tests/plain/gebilorn_plain.py
in float64.
"""
from __future__ import annotations

import torch

from tests.bapavik_cases import BACKENDS, make_engine, runtime_for, tolerance, write_model  # noqa: F401
from tests.bapavik_cases import compare_rows as _compare_rows
from tests.plain import gebilorn_plain as P


def ATT(heads, kv, dim, vdim, scale, size, keep, base, dims, scaling=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size, "keep_first": keep},
         "rot": {"base": base, "dims": dims}}
    if scaling is not None:
        m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    if keep is None:
        del m["mask"]["keep_first"]         # a file may leave the kept first tokens out: none
    if size is None:
        del m["mask"]                       # and the mask: every earlier position is seen
    if dims is None:
        del m["rot"]                        # and the rotation
    return m


def PAR(lh, lkv, ldim, lvdim, lscale, conv, size, rh, rdim, rvdim, tau, left_scale, right_scale):
    return {"left": {"heads": lh, "kv_heads": lkv, "dim": ldim, "vdim": lvdim, "scale": lscale, "conv": conv, "mask": {"size": size}},
            "right": {"heads": rh, "dim": rdim, "vdim": rvdim, "tau": tau}, "left_scale": left_scale, "right_scale": right_scale}


LAT = lambda heads, dim, rot, vdim, rank, q_rank, scale, base: {
    "heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank, "scale": scale, "rot": {"base": base, "dims": rot}}
DENSE = lambda ff: {"kind": "dense", "ff": ff}


def MOE(experts, top, ff, scale=None, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if scale is not None:
        f["router"]["scale"] = scale
    if shared is not None:
        f["shared"] = {"ff": shared}
    return f


BIGRAM = lambda buckets, prev, cur: {"buckets": buckets, "mul_prev": prev, "mul_cur": cur}

# Sizes differ between layers and from each other wherever the design allows: value heads smaller and larger than the
# query/key heads; one key/value head per query head, one for two and one for all; rotation of a part of a head and of
# all of it, with frequencies that fall into all three bands of the scaling rule, and without scaling; windows shorter
# than a page and longer than several; no kept first tokens, fewer than a page holds and more; convolutions of two,
# three and four taps; state heads with more and fewer value than key channels; experts with one choice per token and
# with all of them, with and without a scale and a shared expert; every kind of feed-forward behind every kind of mixer,
# and none; the three mixers in every order; with and without the pair table and the cap on the logits.
CONFIGS = {
    "a": {"architecture": "Gebilorn", "width": 64, "vocab": 150, "norm": {"eps": 1e-5}, "logit_softcap": 12.0,
          "embedding": {"scale": 6.0, "bigram": BIGRAM(61, 7, 13)}, "layers": [
        {"type": "parallel", "mixer": PAR(4, 2, 24, 16, 0.2, 3, 20, 2, 16, 24, 8.0, 0.7, 0.6), "mlp": MOE(6, 2, 32, 1.75, shared=48)},
        {"type": "attention", "mixer": ATT(4, 2, 24, 16, 0.2, 20, 3, 10000.0, 16, (4.0, 1.0, 4.0, 64)), "mlp": DENSE(96)},
        {"type": "latent_attention", "mixer": LAT(4, 16, 8, 24, 40, 28, 0.2, 10000.0), "mlp": None},
        {"type": "attention", "mixer": ATT(2, 2, 16, 32, 0.3, 33, 5, 500.0, 16), "mlp": MOE(4, 1, 48)},
        {"type": "parallel", "mixer": PAR(2, 2, 16, 16, 0.25, 2, 9, 4, 8, 8, 3.0, 1.0, 1.0), "mlp": DENSE(80)},
    ]},
    # sizes that are multiples of nothing: no vector load, no tensor-core tile and no padded head fits them exactly
    "o": {"architecture": "Gebilorn", "width": 100, "vocab": 131, "norm": {"eps": 3e-5}, "logit_softcap": 40.0,
          "embedding": {"scale": 5.5, "bigram": BIGRAM(1000, 131, 1)}, "layers": [
        {"type": "latent_attention", "mixer": LAT(5, 12, 6, 10, 30, 17, 0.22, 3000.0), "mlp": MOE(5, 3, 22, 0.8, shared=30)},
        {"type": "attention", "mixer": ATT(6, 1, 20, 12, 0.25, 7, None, 3000.0, 10, (8.0, 1.0, 4.0, 32)), "mlp": DENSE(70)},
        {"type": "parallel", "mixer": PAR(6, 3, 12, 20, 0.3, 4, 50, 3, 12, 20, 20.0, 0.5, 1.25), "mlp": None},
        {"type": "attention", "mixer": ATT(3, 3, 12, 20, 0.35, None, None, None, None), "mlp": MOE(3, 3, 30, 2.0)},
    ]},
    # no pair table and no cap; a window far longer than the pages, many kept tokens
    "q": {"architecture": "Gebilorn", "width": 48, "vocab": 97, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "layers": [
        {"type": "attention", "mixer": ATT(6, 3, 8, 8, 0.5, 64, 17, 100.0, 8, (2.0, 1.0, 8.0, 16)), "mlp": MOE(7, 2, 16, shared=16)},
        {"type": "parallel", "mixer": PAR(3, 1, 16, 8, 0.3, 3, 44, 1, 32, 16, 1.0, 0.9, 0.4), "mlp": DENSE(64)},
        {"type": "latent_attention", "mixer": LAT(3, 8, 8, 16, 24, 12, 0.25, 100.0), "mlp": MOE(4, 4, 16, 0.5)},
    ]},
}
RANKS = {"a": 8, "o": 5, "q": 12}

# Layers as wide as a real model's: heads of 64 and 128, latent rows of 192 + 64, experts and dense widths that are
# multiples of 64, so the bfloat16 products run on the tensor-core tiles and the attention on its widest head sizes.
CONFIGS["wide"] = {"architecture": "Gebilorn", "width": 512, "vocab": 300, "norm": {"eps": 1e-5}, "logit_softcap": 25.0,
                   "embedding": {"scale": 12.0, "bigram": BIGRAM(523, 101, 19)}, "layers": [
    {"type": "attention", "mixer": ATT(8, 2, 128, 128, 0.06, 96, 4, 200000.0, 64, (4.0, 1.0, 8.0, 1024)), "mlp": MOE(8, 2, 128, 1.25, shared=128)},
    {"type": "parallel", "mixer": PAR(8, 4, 64, 64, 0.125, 4, 80, 4, 64, 128, 12.0, 0.75, 0.55), "mlp": DENSE(1024)},
    {"type": "latent_attention", "mixer": LAT(8, 64, 64, 64, 192, 256, 0.088, 10000.0), "mlp": MOE(8, 2, 128, 1.25)},
]}
RANKS["wide"] = 16


def make_weights(cfg: dict, seed: int, rank: int = 8, expert_gain: float = 1.0):
    """float32 weights by name, sized so that every layer's output matters."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in P.tensor_shapes(cfg, rank).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1",) or name == "final.norm":
            t = 0.2 * torch.randn(shape, generator=g)              # (the stored weight is its distance from one)
        elif leaf == "norm":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif leaf == "sink":
            t = torch.randn(shape, generator=g) * 1.5
        elif leaf == "b":
            t = torch.randn(shape, generator=g) * 0.3
        elif leaf == "conv":
            t = torch.randn(shape, generator=g) * 0.6
        elif leaf == "embed":
            t = torch.randn(shape, generator=g) / cfg["embedding"]["scale"]
        elif leaf == "bigram":
            t = torch.randn(shape, generator=g) * 0.7
        else:
            t = torch.randn(shape, generator=g) * 1.5 / shape[-1] ** 0.5
        if leaf == "down" and ".e" in name:
            t = t * expert_gain
        w[name] = t.bfloat16().float()          # values that a bfloat16 file holds exactly
    return w


def plain_logits(w, cfg, tokens, streams=None):
    with torch.no_grad():
        return P.forward(tokens, {k: v.double() for k, v in w.items()}, cfg, streams).float()


def compare_rows(got, plain, backend, allow: int = 0) -> float:
    """As ``bapavik_cases.compare_rows``; in bfloat16 up to ``allow`` rows (at least one in twenty) may move further: a
    router's choice scores can lie closer than the rounding of its input, and the other expert then changes the row."""
    if backend[1] == "float32":
        return _compare_rows(got, plain, backend)
    bad, worst = 0, 0.0
    for (rid, pos), row in got.items():
        ref = plain[rid][pos]
        assert bool(torch.isfinite(row).all()), f"request {rid!r} position {pos}: not finite"
        d = row - ref
        e = float((d - d.mean()).pow(2).mean().sqrt() / (ref - ref.mean()).pow(2).mean().sqrt())
        worst = max(worst, e)
        bad += e > 0.08
    assert bad <= max(allow, len(got) // 20), f"{bad} of {len(got)} rows differ by more than 8 % (worst {worst:.3f})"
    return worst
