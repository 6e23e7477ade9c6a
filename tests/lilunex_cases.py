"""Shared by the Lilunex tests: small configurations of their own, seeded weights, engines on either backend.

Two backends: "emu" runs the engine's own parts, cache manager and step function on the CPU over the torch stand-ins of
tests/emu_kernels.py (no GPU needed, float32); "cuda" runs the real kernels. The oracle is tests/plain/lilunex_plain.py
in float64.
"""
from __future__ import annotations

import torch

from tests.bapavik_cases import BACKENDS, make_engine, runtime_for, tolerance, write_model  # noqa: F401
from tests.bapavik_cases import compare_rows as _compare_rows
from tests.plain import lilunex_plain as P

WKV = lambda heads, dim: {"heads": heads, "dim": dim}
DELTA = lambda heads, kv, dim, vdim, conv: {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def ATT(heads, kv, dim, vdim, scale, size, keep, base, dims, factor, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size, "keep_first": keep},
         "rot": {"base": base, "dims": dims, "scaling": {"factor": factor}}}
    if factor is None:
        del m["rot"]["scaling"]             # a file may leave the scaling out: frequencies as they are
    if keep is None:
        del m["mask"]["keep_first"]         # and the kept first tokens: none
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


DENSE = lambda ff: {"kind": "dense", "ff": ff}


def MOE(experts, identity, top, ff, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}
    if shared is not None:
        f["shared"] = {"ff": shared}
    return f


# Sizes differ between layers and from each other wherever the design allows: value heads smaller and larger than the
# query/key heads; one key/value head per query head, one for two and one for all; rotation of a part of a head and of all
# of it, with and without scaled frequencies; windows shorter than a page and longer than several; no kept first tokens,
# fewer than a page holds and more; a layer that reads another layer's keys through a longer window and more kept tokens
# than the owner's; convolutions of two, three and four taps; experts with one choice per token and with all of them,
# with and without identity outputs and a shared expert; every kind of feed-forward behind every kind of mixer, and none.
CONFIGS = {
    "a": {"architecture": "Lilunex", "width": 64, "vocab": 150, "norm": {"eps": 1e-5}, "embedding": {"scale": 8.0}, "layers": [
        {"type": "wkv", "mixer": WKV(2, 16), "mlp": MOE(6, 2, 2, 32, shared=48)},
        {"type": "attention", "mixer": ATT(4, 2, 24, 16, 0.2, 20, 3, 10000.0, 16, 2.0), "mlp": DENSE(96)},
        {"type": "delta", "mixer": DELTA(4, 2, 16, 24, 4), "mlp": None},
        {"type": "attention", "mixer": ATT(4, 2, 24, 16, 0.3, 33, 5, 10000.0, 16, 2.0, kv_from=1), "mlp": MOE(4, 0, 1, 48)},
        {"type": "delta", "mixer": DELTA(2, 2, 32, 16, 2), "mlp": DENSE(80)},
    ]},
    # sizes that are multiples of nothing: no vector load, no tensor-core tile and no padded head fits them exactly
    "o": {"architecture": "Lilunex", "width": 100, "vocab": 131, "norm": {"eps": 3e-5}, "embedding": {"scale": 5.5}, "layers": [
        {"type": "attention", "mixer": ATT(6, 1, 20, 12, 0.3, 7, None, 3000.0, 10, None), "mlp": MOE(5, 3, 3, 22, shared=30)},
        {"type": "wkv", "mixer": WKV(5, 12), "mlp": DENSE(70)},
        {"type": "attention", "mixer": ATT(6, 1, 20, 12, 0.25, 50, 9, 3000.0, 10, None, kv_from=0), "mlp": None},
        {"type": "delta", "mixer": DELTA(3, 3, 12, 20, 3), "mlp": MOE(3, 1, 4, 30)},
    ]},
    "q": {"architecture": "Lilunex", "width": 48, "vocab": 97, "norm": {"eps": 1e-6}, "layers": [
        {"type": "delta", "mixer": DELTA(6, 2, 8, 8, 2), "mlp": MOE(7, 1, 2, 16, shared=16)},
        {"type": "attention", "mixer": ATT(6, 3, 8, 8, 0.35, 64, 17, 100.0, 8, 8.0), "mlp": DENSE(64)},
        {"type": "wkv", "mixer": WKV(1, 32), "mlp": None},
    ]},
}
RANKS = {"a": 8, "o": 5, "q": 12}       # width of the wkv decay's two-step projection (the weight file decides it)

# Layers as wide as a real model's: heads of 64 and 128, expert and dense widths that are multiples of 64, so the bfloat16
# products run on the tensor-core tiles and the attention on its widest head sizes.
CONFIGS["wide"] = {"architecture": "Lilunex", "width": 512, "vocab": 300, "norm": {"eps": 1e-5}, "embedding": {"scale": 12.0}, "layers": [
    {"type": "attention", "mixer": ATT(8, 2, 128, 64, 0.088, 160, 6, 50000.0, 64, 2.0), "mlp": MOE(8, 2, 2, 128, shared=256)},
    {"type": "wkv", "mixer": WKV(8, 64), "mlp": DENSE(1024)},
    {"type": "delta", "mixer": DELTA(8, 4, 64, 128, 4), "mlp": MOE(8, 0, 2, 128)},
    {"type": "attention", "mixer": ATT(8, 2, 128, 64, 0.088, 300, 70, 50000.0, 64, 2.0, kv_from=0), "mlp": DENSE(1024)},
]}
RANKS["wide"] = 32


def with_ranks(cfg: dict, rank: int) -> dict:
    """The configuration with the decay rank written into every wkv mixer (for the plain implementation's list of shapes)."""
    import copy

    c = copy.deepcopy(cfg)
    for layer in c["layers"]:
        if layer["type"] == "wkv":
            layer["mixer"]["rank"] = rank
    return c


def make_weights(cfg: dict, seed: int, rank: int = 8):
    """float32 weights by name, sized so that every layer's output matters, decays stay away from 0 and 1, the router's
    softmax is not flat and the choice bias really changes choices."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda shape, std=1.0: torch.randn(shape, generator=g) * std
    w = {}
    for name, shape in P.tensor_shapes(with_ranks(cfg, rank)).items():
        leaf = name.split(".")[-1]
        if leaf == "alpha":
            t = 0.5 + 0.5 * torch.rand(shape, generator=g)
        elif leaf == "b" and len(shape) == 1 and ".mix." in name and name.split(".")[-2] in ("q", "k", "v", "o"):
            t = rnd(shape, 0.2)
        elif leaf == "b" and len(shape) == 1:
            t = rnd(shape, 0.1)                                    # a norm's bias
        elif leaf in ("norm", "norm1", "norm2", "norm1b", "norm2b"):
            t = 1.0 + rnd(shape, 0.2)
        elif leaf in ("r", "k", "v", "g", "w") and ".mu." in name:
            t = torch.rand(shape, generator=g)
        elif leaf == "w0":
            t = -1.0 + rnd(shape, 0.7)
        elif leaf == "u":
            t = rnd(shape, 0.5)
        elif leaf in ("A_log", "dt_bias"):
            t = rnd(shape, 0.5)
        elif leaf == "sink":
            t = rnd(shape, 1.5)
        elif leaf == "conv":
            t = rnd(shape, 0.6)
        elif leaf == "correction":
            t = rnd(shape, 0.15)
        elif leaf == "router":
            t = rnd(shape, 3.0 / shape[-1] ** 0.5)
        elif leaf == "embed":
            t = rnd(shape) / (cfg["embedding"]["scale"] if cfg.get("embedding") else 1.0)
        else:
            t = rnd(shape, 1.5 / shape[-1] ** 0.5)
        w[name] = t.bfloat16().float()          # values that a bfloat16 file holds exactly
    return w


def plain_logits(w, cfg, tokens, layers_out=None):
    with torch.no_grad():
        return P.forward(cfg, w, tokens, torch.float64, layers_out).float()


def compare_rows(got, plain, backend) -> float:
    """Every collected row against the plain logits. float32: every element within ``tolerance``. bfloat16: a row's error is
    the root mean square of its difference (means taken off) over that of the plain row, a few percent from the roundings
    to 8 bits. A router's choice is a discontinuity: where two choice scores lie closer than the rounding noise the engine
    in bfloat16 may take the other expert, and that token's row (and, through the recurrent states and cached keys, rows
    after it) moves by more. So in bfloat16 one row in twenty may exceed the bound, none by far; float32 is strict."""
    if backend[1] == "float32":
        return _compare_rows(got, plain, backend)
    errors = []
    for (rid, pos), row in got.items():
        ref = plain[rid][pos]
        assert bool(torch.isfinite(row).all()), f"request {rid!r} position {pos}: not finite"
        d = row - ref
        errors.append(float((d - d.mean()).pow(2).mean().sqrt() / (ref - ref.mean()).pow(2).mean().sqrt()))
    over = [e for e in errors if e > 0.08]
    assert len(over) <= max(1, len(errors) // 20) and max(errors) < 0.4, f"{len(over)} of {len(errors)} rows over the bound, worst {max(errors):.3f}"
    return max(errors)
