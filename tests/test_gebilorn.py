"""The Gebilorn decoder in the engine against the plain implementation of tests/plain/gebilorn_plain.py.

Every test runs on the CPU over the torch stand-ins of the kernels (which checks the parts, the cache manager, the step
function and the scheduler) and, marked gpu, on the real kernels in float32 and bfloat16.
"""
import copy
import json
import os
import subprocess
import sys

import pytest
import torch

from serve_b200.cache import CacheManager
from serve_b200.config import ConfigError, PartSpec, build_spec, config_from_dict
from serve_b200.parts import build_part
from tests import helpers
from tests.gebilorn_cases import (ATT, BACKENDS, BIGRAM, CONFIGS, DENSE, LAT, MOE, PAR, RANKS, compare_rows, make_engine, make_weights,
                                  plain_logits, runtime_for, write_model)
from tests.plain import gebilorn_plain as P
from tests.test_bapavik import _ctx, _run_part, _tol

LENGTHS = {"a": [1, 5, 23, 49, 75, 130], "o": [3, 40, 90, 17], "q": [2, 9, 31, 64, 101]}
PAGE = {"a": 8, "o": 4, "q": 16}
F64 = lambda w: {k: v.double() for k, v in w.items()}


# ---- configuration and description ----------------------------------------------------------------------------
def test_configuration_is_read_from_the_file_and_describes_every_layer():
    for name, raw in CONFIGS.items():
        cfg = config_from_dict(copy.deepcopy(raw))
        assert type(cfg).__name__ == "GebilornConfig" and cfg.width == raw["width"] and cfg.vocab == raw["vocab"]
        assert cfg.logit_softcap == raw.get("logit_softcap") and (cfg.bigram is None) == ("bigram" not in raw["embedding"])
        spec = build_spec(cfg)
        assert spec.embedding.kind == ("pair_table" if cfg.bigram else "table") and spec.head.params["tied_to"] == "embed"
        assert len(spec.layers) == len(raw["layers"]) == len(spec.schedule)
        kinds = {"attention": "rotary_sink_attention", "parallel": "parallel", "latent_attention": "latent_attention"}
        for layer, ls in zip(raw["layers"], spec.layers):
            assert ls.block.kind == "parallel_residual" and ls.parts["mixer"].kind == kinds[layer["type"]]
            assert ("feed_forward" in ls.parts) == (layer["mlp"] is not None)
            p = ls.parts["mixer"].params
            if layer["type"] == "attention":
                mask = layer["mixer"].get("mask") or {}
                assert p["window"] == mask.get("size") and p["keep_first"] == (mask.get("keep_first") or 0) and p["gate"] == "element"
            if layer["type"] == "parallel":
                assert p["left"].params["conv"] == layer["mixer"]["left"]["conv"] and p["right"].params["tau"] == layer["mixer"]["right"]["tau"]
            if layer["mlp"] and layer["mlp"]["kind"] == "moe":
                assert ls.parts["feed_forward"].params["weight_scale"] == (layer["mlp"]["router"].get("scale") or 1.0)
        assert config_from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("breaker", [
    lambda c: c["layers"][0].update(type="conv"),
    lambda c: c["layers"][1]["mixer"].pop("scale"),
    lambda c: c["layers"][1]["mixer"].update(heads=3),
    lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7),
    lambda c: c["layers"][1]["mixer"]["rot"].update(dims=26),
    lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("original"),
    lambda c: c["layers"][1]["mixer"]["mask"].update(size=0),
    lambda c: c["layers"][0]["mixer"]["left"].update(conv=0),
    lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(keep_first=2),
    lambda c: c["layers"][0]["mixer"]["right"].update(tau=0.0),
    lambda c: c["layers"][0]["mixer"].pop("right_scale"),
    lambda c: c["layers"][2]["mixer"].pop("q_rank"),
    lambda c: c["layers"][2]["mixer"].update(rot_dim=7),
    lambda c: c["layers"][0]["mlp"]["router"].update(top=9),
    lambda c: c["layers"][0]["mlp"].update(kind="sparse"),
    lambda c: c["embedding"]["bigram"].update(buckets=0),
    lambda c: c["norm"].update(eps=0.0),
    lambda c: c.update(logit_softcap=-1.0),
    lambda c: c.pop("vocab"),
])
def test_configuration_refuses_what_it_cannot_run(breaker):
    raw = copy.deepcopy(CONFIGS["a"])
    breaker(raw)
    with pytest.raises(ConfigError):
        config_from_dict(raw)


# ---- whole models ---------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """{config name: {dtype: (weights, requests, plain logits, model folder)}}."""
    out = {}
    for name in LENGTHS:
        cfg = CONFIGS[name]
        reqs = {f"r{i}": helpers.random_tokens(cfg["vocab"], n, seed=20 + i) for i, n in enumerate(LENGTHS[name])}
        w = make_weights(cfg, 100 + len(name), RANKS[name], expert_gain=0.5)
        plain = {rid: plain_logits(w, cfg, toks) for rid, toks in reqs.items()}
        out[name] = {dt: (w, reqs, plain, write_model(str(tmp_path_factory.mktemp(f"{name}-{dt}")), cfg, w, getattr(torch, dt)))
                     for dt in ("float32", "bfloat16")}
    return out


def test_plain_layers_feed_one_another(models):
    """The oracle's own premise: every layer changes the residual stream, the last positions depend on the first token, and
    a token's row depends on the token before it (through the pair table) where the model has one."""
    for name in LENGTHS:
        w, reqs, plain, _ = models[name]["float32"]
        cfg, toks = CONFIGS[name], reqs["r2"]
        layers = []
        plain_logits(w, cfg, toks, layers)
        for a, b in zip(layers, layers[1:]):
            assert float((a - b).abs().max()) > 1e-2
        other = [(toks[0] + 1) % cfg["vocab"]] + toks[1:]
        assert float((plain_logits(w, cfg, other)[-1] - plain["r2"][-1]).abs().max()) > 1e-4
        if "bigram" in cfg["embedding"]:
            x = P.embed(toks[:3], F64(w), cfg)
            y = P.embed([other[0]] + toks[1:3], F64(w), cfg)
            assert float((x[1] - y[1]).abs().max()) > 1e-3 and float((x[2] - y[2]).abs().max()) == 0.0


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("name", ["a", "o", "q"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "pairs", "single_tokens"])
def test_cuts_match_plain(models, name, backend, cut):
    w, reqs, plain, folder = models[name][backend[1]]
    page = PAGE[name]
    eng = make_engine(folder, backend, page, num_pages=-(-160 // page) * 2, graphs=(cut == "tail_decode"))
    if cut == "single_tokens":
        steps = helpers.trace_tail_decode({k: v for k, v in reqs.items() if len(v) <= 50}, tail=10 ** 6)
    else:
        make = {"whole": helpers.trace_whole, "tail_decode": lambda r: helpers.trace_tail_decode(r, tail=40),
                "portions": lambda r: helpers.trace_portions(r, sizes=(7, 2, 19, 1, 3, 2, 33, 5, 2, 11)),
                "pairs": lambda r: helpers.trace_portions({k: v for k, v in r.items() if len(v) <= 80}, sizes=(2,))}[cut]
        steps = make(reqs)
    with torch.inference_mode():
        got = helpers.replay(eng, steps)
    eng.kernels.check_errors()
    compare_rows(got, plain, backend)
    eng.cache.check()
    assert eng.cache.live == 0


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("name", ["a", "o", "q"])
def test_mixed_batches_with_pages_and_slots_used_again(models, name, backend):
    """Unequal requests side by side, portions beside single tokens, fewer slots and pages than the requests need in
    all: every row must equal the request run alone. Pages are poisoned first, so that a page that is read without
    having been written shows; a slot's states (matrix states, convolution tails, the previous token) are the next
    request's whoever had the slot before."""
    w, reqs, plain, folder = models[name][backend[1]]
    page = PAGE[name]
    steps = helpers.trace_mixed(reqs, live=3, seed=7)
    need = helpers.tokens_needed(steps, page) // page
    assert need < sum(-(-len(t) // page) for t in reqs.values())
    eng = make_engine(folder, backend, page, num_pages=need, max_slots=3, context=160)
    for view in eng.stepper.views:
        if view is not None and view.k is not None:
            view.k.fill_(float("nan"))
            view.v.fill_(float("nan"))
    with torch.inference_mode():
        got = helpers.replay(eng, steps)
    eng.kernels.check_errors()
    compare_rows(got, plain, backend)
    eng.cache.check()
    assert eng.cache.live == 0 and eng.cache.free_slots == 3
    assert max(g.pool.high_water for g in eng.cache.groups) <= need


@pytest.mark.parametrize("backend", BACKENDS)
def test_long_decoding_side_by_side(models, backend):
    """Two requests decoded one token at a time for 120 steps after short prompts (from CUDA graphs on the GPU): the windows
    of 64 and 40 pass over decoded tokens, pages are crossed and given back many times, the kept first tokens stay, the
    matrix state and the previous token travel from replay to replay."""
    cfg = CONFIGS["q"]
    w, _, _, folder = models["q"][backend[1]]
    seqs = {f"d{i}": helpers.random_tokens(cfg["vocab"], 140 - 9 * i, seed=60 + i) for i in range(2)}
    plain = {rid: plain_logits(w, cfg, toks) for rid, toks in seqs.items()}
    eng = make_engine(folder, backend, 16, num_pages=20, graphs=True)
    steps = [{"step": 0, "entries": [{"id": rid, "tokens": t[:11 + 6 * i], "want": [10 + 6 * i]} for i, (rid, t) in enumerate(seqs.items())], "end": []}]
    at = {rid: 11 + 6 * i for i, rid in enumerate(seqs)}
    while any(at[rid] < len(seqs[rid]) for rid in seqs):
        entries = [{"id": rid, "tokens": [t[at[rid]]], "want": [0]} for rid, t in seqs.items() if at[rid] < len(t)]
        for e in entries:
            at[e["id"]] += 1
        steps.append({"step": len(steps), "entries": entries, "end": []})
    with torch.inference_mode():
        got = helpers.replay(eng, steps)
    eng.kernels.check_errors()
    if backend[0] == "cuda":
        assert eng.stepper.launched_graphs > 80
    compare_rows(got, plain, backend)


@pytest.mark.parametrize("backend", BACKENDS)
def test_greedy_generation_through_the_scheduler(models, backend):
    """generate(): the engine's own entry point, scheduler and sampler; the sampled token stays on the device, so the pair
    table's row comes from two tokens the host never sent. Every generated token must be (within the tolerance) the best
    one of the plain model given the tokens before it."""
    from serve_b200.run import Request, generate

    cfg = CONFIGS["a"]
    w, reqs, _, folder = models["a"][backend[1]]
    eng = make_engine(folder, backend, 8, num_pages=40, max_slots=3, budget=32)
    prompts = [reqs["r1"], reqs["r2"], reqs["r3"][:30], reqs["r0"]]
    out = generate(eng, [Request(torch.tensor(p), len(p), 12) for p in prompts], temperature=0.0, eos_token_id=None)
    for p, r in zip(prompts, out):
        new = r.generated_tokens.tolist()
        assert len(new) == 12
        logits = plain_logits(w, cfg, p + new)
        tol = float(logits.abs().max()) * (2e-4 if backend[1] == "float32" else 2.0 ** -4)
        for i, tok in enumerate(new):
            row = logits[len(p) - 1 + i]
            assert float(row[tok]) >= float(row.max()) - 2 * tol, f"token {i} of a request is not the plain model's choice"
    assert eng.cache.live == 0


# ---- each mechanism alone ---------------------------------------------------------------------------------------
CUTS = [[57], [30, 1, 1, 2, 5, 17, 1], [1] * 57]


def _single(kind, mixer=None, mlp=None, width=64):
    """A one-layer configuration around the mechanism under test."""
    return {"architecture": "Gebilorn", "width": width, "vocab": 50, "norm": {"eps": 1e-5}, "embedding": {"scale": 4.0},
            "layers": [{"type": kind, "mixer": mixer, "mlp": mlp}]}


def _plain_mixer(kind, x, w64, m, eps, p="l0.mix."):
    return P.mixer(x, w64, p, {"type": kind, "mixer": m}, eps)


def _mixer_alone(backend, cfg, cuts, seed=5, x=None, tweak=None, page=8, loose=1.0, rank=8, side=None):
    from serve_b200.models.gebilorn import _mixer_spec

    layer = cfg["layers"][0]
    w = make_weights(cfg, seed, rank)
    if tweak is not None:
        tweak(w, "l0.mix.")
    if x is None:
        x = torch.randn(sum(cuts), cfg["width"], generator=torch.Generator().manual_seed(seed + 1))
    x = x.bfloat16().float()
    spec = _mixer_spec(layer["type"], layer["mixer"], cfg["width"], cfg["norm"]["eps"], "l0.mix.")
    m, eps = layer["mixer"], cfg["norm"]["eps"]
    if side is not None:            # one side of a parallel pair, as a mixer of its own
        spec = spec.params[side]
        want = (P.conv_window_attention(x.double(), F64(w), "l0.mix.left.", m["left"]) if side == "left" else
                P.decaying_state_mixer(x.double(), F64(w), "l0.mix.right.", m["right"], eps)).float()
    else:
        want = _plain_mixer(layer["type"], x.double(), F64(w), m, eps).float()
    got = _run_part(backend, "mixer", spec, w, x, cuts, page=page)
    torch.testing.assert_close(got, want, atol=_tol(backend, want) * loose, rtol=0)
    return got, want, w


# Also: no rotation, no mask and no kept tokens in the file; a window of one key (the query's own) with two kept tokens; a
# window as long as the kept tokens; value heads wider than the keys'; one head; rotation of the whole head; frequencies in
# all three bands of the scaling rule (32 positions "original": waves shorter than 8, longer than 32, and between).
ATTS = [ATT(4, 2, 24, 16, 0.2, 20, 3, 10000.0, 16, (4.0, 1.0, 4.0, 32)), ATT(6, 1, 20, 12, 0.3, 7, None, 3000.0, 10),
        ATT(6, 3, 8, 8, 0.5, 64, 17, 100.0, 8, (8.0, 2.0, 16.0, 64)), ATT(2, 2, 16, 40, 0.25, 9, 9, 500.0, 16),
        ATT(3, 1, 32, 32, 0.12, 1, 2, 7000.0, 32, (2.0, 1.0, 4.0, 16)), ATT(1, 1, 16, 16, 0.3, None, None, None, None)]
PARS = [PAR(4, 2, 24, 16, 0.2, 3, 20, 2, 16, 24, 8.0, 0.7, 0.6), PAR(6, 3, 12, 20, 0.3, 4, 50, 3, 12, 20, 20.0, 0.5, 1.25),
        PAR(3, 1, 16, 8, 0.3, 2, 5, 1, 32, 16, 1.0, 0.9, 0.4), PAR(2, 2, 64, 32, 0.1, 1, 1, 2, 64, 64, 2.5, 1.0, 1.0)]
LATS = [LAT(4, 16, 8, 24, 40, 28, 0.2, 10000.0), LAT(5, 12, 6, 10, 30, 17, 0.22, 3000.0), LAT(3, 8, 8, 16, 24, 12, 0.25, 100.0),
        LAT(1, 24, 4, 16, 20, 50, 0.19, 500.0), dict(LAT(2, 16, 16, 16, 24, 12, 0.2, 1000.0), rot={"base": 1000.0}),      # the file may leave rot.dims out
        dict(LAT(2, 16, 16, 16, 24, 12, 0.2, 1000.0), rot={"base": 1000.0, "dims": 8}),                                   # or turn a part of the rotated part only
        LAT(2, 16, 8, 16, 264, 20, 0.2, 100.0)]      # a latent row wider than the attention kernels take: keys and values cached per head
WIDTHS = (64, 100, 48, 40, 72, 56, 64, 80)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("cuts", CUTS, ids=["whole", "portions", "tokens"])
@pytest.mark.parametrize("which", range(len(ATTS)))
def test_attention_alone(backend, cuts, which):
    _mixer_alone(backend, _single("attention", ATTS[which], width=WIDTHS[which]), cuts)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("cuts", CUTS, ids=["whole", "portions", "tokens"])
@pytest.mark.parametrize("side", ["left", "right", None], ids=["convolved-attention", "decaying-state", "pair"])
@pytest.mark.parametrize("which", range(len(PARS)))
def test_parallel_pair_and_each_side_alone(backend, cuts, which, side):
    """The convolved window attention (also: one tap, which is no convolution and keeps no state; a window of one key), the
    decaying matrix state (also: one head; more and fewer value than key channels) and their scaled sum."""
    _mixer_alone(backend, _single("parallel", PARS[which], width=WIDTHS[which]), cuts, rank=(8, 5, 12, 3)[which], side=side, loose=2.0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("cuts", CUTS, ids=["whole", "portions", "tokens"])
@pytest.mark.parametrize("which", range(len(LATS)))
def test_latent_attention_alone(backend, cuts, which):
    _mixer_alone(backend, _single("latent_attention", LATS[which], width=WIDTHS[which]), cuts, loose=2.0)


def test_rotation_frequencies_fall_into_every_band():
    """The oracle's frequencies: kept, divided by the factor, and blended between, and the engine's table equals them."""
    from serve_b200.parts.rotary import rotary_inv_freq

    rot = {"base": 10000.0, "dims": 16, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}}
    plain = P.frequencies(rot)
    raw = [10000.0 ** (-2.0 * i / 16) for i in range(8)]
    kinds = {"kept" if f == r else "slowed" if abs(f - r / 4.0) < 1e-12 else "between" for f, r in zip(plain, raw)}
    assert kinds == {"kept", "slowed", "between"}
    mine = rotary_inv_freq(16, 10000.0, {"factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 32})
    torch.testing.assert_close(mine.double(), torch.tensor(plain, dtype=torch.float64), rtol=1e-6, atol=0)


def _ff_alone(backend, f, width, seed=11, tweak=None, n=40):
    from serve_b200.models.gebilorn import _feed_forward_spec

    cfg = _single("attention", ATTS[0], f, width)
    w = make_weights(cfg, seed)
    if tweak is not None:
        tweak(w)
    x = torch.randn(n, width, generator=torch.Generator().manual_seed(seed + 1)).bfloat16().float()
    got = _run_part(backend, "feed_forward", _feed_forward_spec(f, width, "l0.mlp."), w, x, [n - 7, 1, 6])
    want = P.feed_forward(x.double(), F64(w), "l0.mlp.", f).float()
    return got, want, w, x


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("ff,width", [(96, 64), (70, 100), (1, 48)])
def test_dense_feed_forward_alone(backend, ff, width):
    got, want, _, _ = _ff_alone(backend, DENSE(ff), width)
    torch.testing.assert_close(got, want, atol=2 * _tol(backend, want), rtol=0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("f,width", [(MOE(6, 2, 32, 1.75, shared=48), 64), (MOE(5, 3, 22, 0.8, shared=30), 100), (MOE(4, 1, 48), 48),
                                     (MOE(3, 3, 30, 2.0), 40), (MOE(1, 1, 16, 3.0, shared=8), 32)])
def test_experts_alone(backend, f, width):
    """Also: one choice, every expert chosen, one expert in all (whose score is 1, so the weight is the scale itself), no
    scale in the file, no shared expert. The router's rows are spread so that no two scores lie within a rounding."""
    def spread(w):
        w["l0.mlp.router"] = (w["l0.mlp.router"] * 3.0).bfloat16().float()
    got, want, w, x = _ff_alone(backend, f, width, tweak=spread)
    if backend[1] == "float32":
        torch.testing.assert_close(got, want, atol=2 * _tol(backend, want), rtol=0)
    else:
        bad = ((got - want).abs().amax(1) > 4 * _tol(backend, want)).sum()
        assert int(bad) <= 2
    # the weights are the scores times the scale, not divided by their sum: doubling the scale doubles the experts' part
    if f["router"].get("scale") and f.get("shared") is None:
        g = copy.deepcopy(f)
        g["router"]["scale"] = 2 * f["router"]["scale"]
        torch.testing.assert_close(P.feed_forward(x.double(), F64(w), "l0.mlp.", g).float(), 2 * want, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("backend", BACKENDS)
def test_shared_expert_gate_is_one_number_per_token(backend):
    """With the routed experts silenced the output is the shared expert times sigmoid(w . h): a gate row scaled up closes the
    shared expert for tokens on one side of it and opens it for the others."""
    f = MOE(4, 2, 16, 1.0, shared=24)

    def tweak(w):
        for e in range(4):
            w[f"l0.mlp.e{e}.down"].zero_()
        w["l0.mlp.shared.sg"] = (w["l0.mlp.shared.sg"] * 40.0).bfloat16().float()
    got, want, w, x = _ff_alone(backend, f, 64, tweak=tweak)
    torch.testing.assert_close(got, want, atol=2 * _tol(backend, want), rtol=0)
    gate = torch.sigmoid(x.double() @ w["l0.mlp.shared.sg"].double().T)[:, 0]
    assert int((gate < 0.05).sum()) > 3 and int((gate > 0.95).sum()) > 3
    assert float(want[gate < 0.01].abs().max()) < 0.02 * float(want.abs().max())


def _embedding_alone(backend, cfg, tokens, cuts, warm):
    """The embedding part over one sequence cut as ``cuts`` says, in a slot another request used before."""
    rt, dev = runtime_for(backend)
    spec = build_spec(config_from_dict(copy.deepcopy(cfg)))
    part = build_part("embedding", spec.embedding, rt)
    w = make_weights(cfg, 3)
    part.load({d.name: w[d.name].to(dev).to(rt.act_dtype) for d in part.tensor_decls()})
    mgr = CacheManager([part.cache_need()], [None], 8, 16, 1, 4096, device=dev, kv_dtype=rt.act_dtype)
    view = mgr.views()[0]
    outs = []
    with torch.inference_mode():
        for rid, toks, cut in (("warm", warm, [len(warm)]), ("r", tokens, cuts)):
            mgr.open(rid)
            at = 0
            for n in cut:
                ctx = _ctx(rt, dev, [n], [at], [mgr.slot(rid)], None, [rid], toks[at: at + n])
                out = part.forward(ctx.tokens, ctx, view)
                if rid == "r":
                    outs.append(out.float().cpu())
                at += n
            mgr.close(rid)
    return torch.cat(outs), P.embed(tokens, F64(w), cfg).float()


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("cuts", [[40], [1] * 40, [2, 1, 17, 1, 1, 18], [1, 39]], ids=["whole", "tokens", "portions", "first-alone"])
@pytest.mark.parametrize("bigram", [BIGRAM(61, 7, 13), BIGRAM(1, 3, 5), BIGRAM(100003, 99991, 1), BIGRAM(17, 0, 1)])
def test_pair_table_embedding(backend, cuts, bigram):
    """The row of a pair depends on the token before, also across the edges of portions; the first token takes the last row,
    whatever the slot held. Also: one bucket, a table larger than vocab^2 with a multiplier near 2^17, a zero multiplier."""
    cfg = _single("attention", ATTS[0])
    cfg["vocab"] = 45000 if bigram["buckets"] > 1000 else 50
    cfg["embedding"]["bigram"] = bigram
    tokens = helpers.random_tokens(cfg["vocab"], 40, seed=9)
    got, want = _embedding_alone(backend, cfg, tokens, cuts, warm=helpers.random_tokens(cfg["vocab"], 9, seed=10))
    torch.testing.assert_close(got, want, atol=1e-5 * float(want.abs().max()), rtol=0)


@pytest.mark.parametrize("backend", BACKENDS)
def test_norm_weight_is_stored_around_zero_and_logits_are_capped(backend):
    rt, dev = runtime_for(backend)
    norm = build_part("norm", PartSpec("rms", {"size": 48, "eps": 1e-5, "weight_name": "n", "offset": 1.0}), rt)
    g = torch.Generator().manual_seed(2)
    wt = (0.3 * torch.randn(48, generator=g)).bfloat16().float()
    norm.load({"n": wt.to(dev).to(rt.act_dtype)})
    x = torch.randn(9, 48, generator=g) * 3.0
    got = norm.forward(x.clone().to(dev), None, None).float().cpu()
    want = P.offset_norm(x.double(), wt.double(), 1e-5).float()
    torch.testing.assert_close(got, want, atol=_tol(backend, want), rtol=0)
    head = build_part("head", PartSpec("linear", {"vocab": 30, "hidden": 48, "name": "head", "tied_to": "e", "softcap": 2.5}), rt)
    table = (torch.randn(30, 48, generator=g)).bfloat16().float()
    head.load({"e": table.to(dev).to(rt.act_dtype)})
    h = torch.randn(5, 48, generator=g).bfloat16().float()
    logits = head.forward(h.to(dev).to(rt.act_dtype), None).float().cpu()
    want = 2.5 * torch.tanh((h.double() @ table.double().T) / 2.5).float()
    assert float(want.abs().max()) > 2.4           # the cap bends these logits
    torch.testing.assert_close(logits, want, atol=_tol(backend, want), rtol=0)


# ---- what a key far away, at a page's or a window's edge, and the sink do ------------------------------------------
def _loud_key(w, p, m, x, at, query_rows, gain=6.0):
    """Make position ``at`` a key that the queries of ``query_rows`` would put nearly all their weight on if they saw it:
    its input is one direction that the key projection maps to a large key, and those queries' inputs share it."""
    direction = torch.zeros(x.shape[1])
    direction[0] = 1.0
    x[at] = direction * gain
    for r in query_rows:
        x[r] = x[r] * 0.3 + direction * gain


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("cuts", [[300], [255, 1, 1, 43], [130] + [1] * 170], ids=["prompt", "portions", "decoded"])
@pytest.mark.parametrize("at,size,keep", [(3, 64, 4), (4, 64, 4), (63, 200, 0), (64, 200, 0), (127, 150, 2), (0, 32, 1), (40, 300, 0)])
def test_one_key_far_back_at_edges_of_pages_windows_and_kept_tokens(backend, cuts, at, size, keep):
    """One key carries a value nobody else has. Queries for which it lies just inside the window (or among the kept first
    tokens) must find it, the next ones must not: both compared with the plain attention, whose difference between the two
    kinds of rows is checked to be large. Pages of 64: the key sits on the last row of a page, the first of the next, and
    hundreds of positions back."""
    m = ATT(2, 1, 16, 16, 0.6, size, keep, 10000.0, 8)
    cfg = _single("attention", m, width=32)
    n = sum(cuts)
    x = torch.randn(n, 32, generator=torch.Generator().manual_seed(at + size)) * 0.5
    _loud_key(None, None, m, x, at, range(at + 1, n))

    def tweak(w, p):
        w[p + "sink"].fill_(-4.0)
        for name in ("q", "k"):
            w[p + name][:, 0] = 0.0
            w[p + name][0::16, 0] = 1.0        # every head's first (rotated) channel listens to the direction
        w[p + "v"][:, 0] = 2.0

    got, want, _ = _mixer_alone(backend, cfg, cuts, x=x, tweak=tweak, page=64)
    seen = [i for i in range(at + 1, n) if P.visible(i, at, size, keep)]
    unseen = [i for i in range(at + 1, n) if not P.visible(i, at, size, keep)]
    assert seen, "the case has no query that sees the key"
    if unseen:      # (against the float32 bound: that run is the sharp one; bfloat16's own bound is of the size of the key's share)
        assert float((want[seen[-1]] - want[unseen[0]]).abs().max()) > 100 * _tol(("", "float32"), want), "the key does not stand out"


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("cuts", [[150], [60, 2, 1, 87], [50] + [1] * 100], ids=["prompt", "portions", "decoded"])
@pytest.mark.parametrize("size", [1, 2, 37, 64, 65])
def test_convolved_attention_window_edges(backend, cuts, size):
    """The left side's plain window: the key at distance size - 1 is seen, the one at distance size is not."""
    m = PAR(2, 1, 16, 16, 0.6, 2, size, 1, 8, 8, 4.0, 1.0, 1.0)
    cfg = _single("parallel", m, width=32)
    n = sum(cuts)
    x = torch.randn(n, 32, generator=torch.Generator().manual_seed(size)) * 0.5
    _loud_key(None, None, m, x, 20, range(21, n))

    def tweak(w, p):
        w[p + "left.sink"].fill_(-4.0)
        for name in ("q", "k", "v"):
            w[p + f"left.{name}.conv"][:, :-1] = 0.0       # the current token's tap only, so that the key stays one position
            w[p + f"left.{name}.conv"][:, -1] = 1.0
            w[p + f"left.{name}.b"].zero_()
        for name in ("q", "k"):
            w[p + f"left.{name}"][:, 0] = 0.0
            w[p + f"left.{name}"][0::16, 0] = 1.0
        w[p + "left.v"][:, 0] = 4.0

    got, want, _ = _mixer_alone(backend, cfg, cuts, x=x, tweak=tweak, page=64, side="left", loose=2.0)
    if 20 + size < n and size > 1:
        assert float((want[20 + size - 1] - want[20 + size]).abs().max()) > 100 * _tol(("", "float32"), want), "the key does not stand out"


@pytest.mark.parametrize("backend", BACKENDS)
def test_the_sink_takes_weight_without_a_value(backend):
    """A large sink shrinks a head's output towards zero, a very negative one leaves the plain softmax; heads differ."""
    m = ATT(2, 2, 16, 16, 0.3, 30, 0, 10000.0, 8)
    cfg = _single("attention", m, width=32)
    outs = {}
    for name, sink in (("open", [6.0, -30.0]), ("closed", [-30.0, -30.0])):
        def tweak(w, p, sink=sink):
            w[p + "sink"] = torch.tensor(sink)
            w[p + "g"].zero_()                               # gates of one half everywhere
            w[p + "o"] = torch.eye(32)                       # the heads' outputs themselves
        outs[name] = _mixer_alone(backend, cfg, [40], tweak=tweak)[1]
    assert float(outs["open"][:, :16].abs().max()) < 0.2 * float(outs["closed"][:, :16].abs().max())
    torch.testing.assert_close(outs["open"][:, 16:], outs["closed"][:, 16:], atol=1e-4, rtol=0)


@pytest.mark.parametrize("backend", BACKENDS)
def test_states_of_a_slot_are_the_next_requests(backend):
    """A parallel pair over a sequence, after another sequence ran in the same slot and was closed: the matrix state and the
    convolution tails of the earlier one (long, and three times as loud) must not reach the later one."""
    from serve_b200.models.gebilorn import _mixer_spec

    m = PARS[0]
    cfg = _single("parallel", m)
    w = make_weights(cfg, 8)
    rt, dev = runtime_for(backend)
    part = build_part("mixer", _mixer_spec("parallel", m, 64, 1e-5, "l0.mix."), rt)
    part.load({d.name: w[d.name].to(dev).to(rt.act_dtype) for d in part.tensor_decls()})
    mgr = CacheManager([part.cache_need()], [None], 8, 16, 1, 256, device=dev, kv_dtype=rt.act_dtype)
    view = mgr.views()[0]
    x = torch.randn(40, 64, generator=torch.Generator().manual_seed(9)).bfloat16().float()
    outs = []
    with torch.inference_mode():
        for rid, rows in (("first", x * 3.0), ("second", x)):
            mgr.open(rid)
            mgr.reserve([(rid, 40)])
            outs.append(part.forward(rows.to(dev).to(rt.act_dtype), _ctx(rt, dev, [40], [0], [mgr.slot(rid)], mgr, [rid]), view).float().cpu())
            mgr.commit(rid, 40)
            mgr.close(rid)
    want = _plain_mixer("parallel", x.double(), F64(w), m, 1e-5).float()
    torch.testing.assert_close(outs[1], want, atol=2 * _tol(backend, want), rtol=0)


def test_the_decaying_state_remembers_and_forgets():
    """The oracle's premise for the recurrent side: with decays near one a token hundreds of positions back still shows in
    the read-out, with decays near zero it is gone after a few tokens."""
    m = PAR(2, 1, 16, 16, 0.3, 2, 4, 2, 16, 16, 1.0, 0.0, 1.0)["right"]
    cfg = _single("parallel", PAR(2, 1, 16, 16, 0.3, 2, 4, 2, 16, 16, 1.0, 0.0, 1.0))
    w = F64(make_weights(cfg, 4))
    x = torch.randn(300, 64, generator=torch.Generator().manual_seed(5)).double()
    y = x.clone()
    y[0] = x[0].roll(7) * 0.5            # (not -x[0]: k v^T would not notice)
    for bias, far in ((9.0, True), (-9.0, False)):
        w["l0.mix.right.a2.b"].fill_(bias)
        d = (P.decaying_state_mixer(x, w, "l0.mix.right.", m, 1e-5) - P.decaying_state_mixer(y, w, "l0.mix.right.", m, 1e-5)).abs().amax(1)
        assert (float(d[299]) > 1e-3) == far and float(d[1]) > 1e-3


# ---- the sizes of a real layer, and the programs a user starts ----------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_as_wide_as_a_real_models(tmp_path, dtype):
    """Heads of 128 and 64, a latent row of 192 + 64, experts and dense widths that are multiples of 64: the products take
    the tensor-core paths, the attention its widest heads; prompts of several hundred tokens, portions and decoded tails."""
    cfg = CONFIGS["wide"]
    w = make_weights(cfg, 31, RANKS["wide"], expert_gain=0.3)
    reqs = {f"r{i}": helpers.random_tokens(cfg["vocab"], n, seed=40 + i) for i, n in enumerate([300, 130, 17])}
    plain = {rid: plain_logits(w, cfg, toks) for rid, toks in reqs.items()}
    folder = write_model(str(tmp_path / "wide"), cfg, w, getattr(torch, dtype))
    backend = ("cuda", dtype)
    for steps, graphs in ((helpers.trace_whole(reqs), False), (helpers.trace_tail_decode(reqs, tail=40), True),
                          (helpers.trace_portions(reqs, sizes=(64, 2, 130, 1, 33)), False)):
        eng = make_engine(folder, backend, 64, num_pages=16, graphs=graphs, budget=1024, context=512)
        with torch.inference_mode():
            got = helpers.replay(eng, steps)
        eng.kernels.check_errors()
        compare_rows(got, plain, backend)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_replay_program_on_a_folder_of_this_design(tmp_path, dtype):
    cfg = CONFIGS["q"]
    w = make_weights(cfg, 17, RANKS["q"], expert_gain=0.5)
    folder = write_model(str(tmp_path / "m"), cfg, w, torch.bfloat16)
    reqs = {f"r{i}": helpers.random_tokens(cfg["vocab"], n, seed=70 + i) for i, n in enumerate([70, 9, 33, 150, 2])}
    wb = {k: v.bfloat16().float() for k, v in w.items()}
    plain = {rid: plain_logits(wb, cfg, toks) for rid, toks in reqs.items()}
    steps = helpers.trace_mixed(reqs, live=4, seed=3)
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", str(out),
                           "--max-tokens", str(helpers.tokens_needed(steps, 64))],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    import numpy as np

    got, at = {}, {}
    for s in steps:
        rows = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        i = 0
        for e in s["entries"]:
            for wnt in e["want"]:
                got[(e["id"], at.get(e["id"], 0) + wnt)] = torch.from_numpy(rows[i].copy())
                i += 1
            at[e["id"]] = at.get(e["id"], 0) + len(e["tokens"])
    compare_rows(got, plain, ("cuda", dtype))


# ---- configurations nobody chose ---------------------------------------------------------------------------------
def _random_config(rng) -> dict:
    """A model of this design drawn at random: widths and vocabularies that are no power of two, 3 to 6 layers in any order with
    at least one of each mixer, head sizes that are and are not multiples of 16, value heads smaller and larger than the keys',
    1 to 4 key/value heads, windows from shorter than a page to longer than the prompts, 0 to 70 kept tokens, partial and full
    rotation with and without scaled frequencies, 2 to 5 taps, 2 to 64 experts with 1 to 8 choices, with and without a shared
    expert, layers without a feed-forward, with and without the pair table and the cap."""
    width = rng.choice([72, 96, 100, 128, 136, 200, 264])

    def att():
        kv = rng.choice([1, 2, 3, 4])
        dim = rng.choice([16, 24, 32, 40, 64, 80, 128])
        m = {"heads": kv * rng.choice([1, 2, 4]), "kv_heads": kv, "dim": dim, "vdim": rng.choice([dim, 16, 48, 72]),
             "scale": rng.choice([2.0, 4.0, 6.0]) / dim}
        if rng.random() < 0.85:
            m["mask"] = {"size": rng.choice([1, 7, 38, 64, 65, 130, 1000])}
            if rng.random() < 0.7:
                m["mask"]["keep_first"] = rng.choice([0, 1, 4, 5, 33, 70])
        if rng.random() < 0.85:
            dims = rng.choice([d for d in (4, 8, 16, 32, 64, 128) if d <= dim] + [dim - dim % 2])
            m["rot"] = {"base": rng.choice([100.0, 10000.0, 500000.0]), "dims": dims}
            if rng.random() < 0.6:
                m["rot"]["scaling"] = {"factor": rng.choice([2.0, 8.0, 32.0]), "low": 1.0, "high": rng.choice([2.0, 4.0]),
                                       "original": rng.choice([16, 64, 2048])}
        return m

    def par():
        kv = rng.choice([1, 2, 4])
        dim, rdim = rng.choice([16, 32, 48, 64]), rng.choice([8, 16, 32, 64, 128])
        return {"left": {"heads": kv * rng.choice([1, 2, 3]), "kv_heads": kv, "dim": dim, "vdim": rng.choice([dim, 16, 80]), "scale": 3.0 / dim,
                         "conv": rng.choice([2, 3, 4, 5]), "mask": {"size": rng.choice([1, 5, 37, 64, 100, 500])}},
                "right": {"heads": rng.choice([1, 2, 3, 4]), "dim": rdim, "vdim": rng.choice([rdim, 16, 64]), "tau": rng.choice([1.0, 4.0, 12.0, 50.0])},
                "left_scale": rng.choice([0.5, 0.8, 1.0]), "right_scale": rng.choice([0.5, 1.0, 1.3])}

    def lat():
        dim, rot = rng.choice([16, 32, 64]), rng.choice([4, 8, 16, 32, 64])
        return {"heads": rng.choice([1, 2, 3, 4, 8]), "dim": dim, "rot_dim": rot, "vdim": rng.choice([dim, 24, 64]),
                "kv_rank": rng.choice([16, 24, 40, 64, 100, 192]), "q_rank": rng.choice([8, 20, 48, 96]), "scale": 1.0 / (dim + rot) ** 0.5,
                "rot": {"base": rng.choice([100.0, 10000.0]), "dims": rot}}

    def mlp():
        r = rng.random()
        if r < 0.15:
            return None
        if r < 0.4:
            return DENSE(rng.choice([64, 90, 128, 333]))
        experts = rng.choice([2, 4, 5, 8, 16, 64])
        return MOE(experts, rng.choice([t for t in (1, 2, 3, 4, 8) if t <= experts]), rng.choice([16, 24, 64]),
                   rng.choice([None, 0.5, 1.5, 2.5]), rng.choice([None, 16, 96]))

    kinds = ["attention", "parallel", "latent_attention"] + [rng.choice(["attention", "parallel", "latent_attention"]) for _ in range(rng.randint(0, 3))]
    rng.shuffle(kinds)
    make = {"attention": att, "parallel": par, "latent_attention": lat}
    cfg = {"architecture": "Gebilorn", "width": width, "vocab": rng.choice([131, 257, 500, 640, 1000]), "norm": {"eps": rng.choice([1e-5, 1e-6])},
           "embedding": {"scale": rng.choice([1.0, 2.5, 8.0])}, "layers": [{"type": k, "mixer": make[k](), "mlp": mlp()} for k in kinds]}
    if rng.random() < 0.8:
        cfg["embedding"]["bigram"] = BIGRAM(rng.choice([1, 61, 523, 4099]), rng.choice([0, 7, 131, 1001]), rng.choice([1, 19, 64]))
    if rng.random() < 0.8:
        cfg["logit_softcap"] = rng.choice([15.0, 25.0, 50.0])
    return cfg


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8])
def test_random_configuration(tmp_path, seed, dtype):
    """Five requests of 2 to 330 tokens in pages of 64, whole, with decoded tails from CUDA graphs, in portions and as mixed batches
    of four live requests on a pool without a spare page, against the plain implementation."""
    import random

    rng = random.Random(seed)
    cfg = _random_config(rng)
    rank = rng.choice([3, 8, 16])
    w = make_weights(cfg, seed, rank, expert_gain=0.3)
    if dtype == "bfloat16":                               # keep routers away from near-ties that 8 bits of the input decide
        for name in w:
            if name.endswith(".router"):
                w[name] = (w[name] * 3.0).bfloat16().float()
    folder = write_model(str(tmp_path / "m"), cfg, w, getattr(torch, dtype))
    lens = [rng.choice([2, 3, 17, 64, 65, 130, 200, 257, 330]) for _ in range(5)]
    reqs = {f"r{i}": helpers.random_tokens(cfg["vocab"], n, seed=seed * 10 + i) for i, n in enumerate(lens)}
    plain = {rid: plain_logits(w, cfg, toks) for rid, toks in reqs.items()}
    backend = ("cuda", dtype)
    cuts = {"whole": helpers.trace_whole, "tail": lambda r: helpers.trace_tail_decode(r, tail=70),
            "portions": lambda r: helpers.trace_portions(r, sizes=(64, 2, 130, 1, 33, 5)), "mixed": lambda r: helpers.trace_mixed(r, live=4, seed=seed)}
    for cut, make in cuts.items():
        steps = make(reqs)
        pages = helpers.tokens_needed(steps, 64) // 64
        eng = make_engine(folder, backend, 64, num_pages=pages, max_slots=4, graphs=(cut == "tail"), budget=max(512, pages * 64), context=pages * 64)
        for v in eng.stepper.views:
            if v is not None and v.k is not None:
                v.k.fill_(float("nan"))
                v.v.fill_(float("nan"))
        with torch.inference_mode():
            got = helpers.replay(eng, steps)
        eng.kernels.check_errors()
        try:
            compare_rows(got, plain, backend, allow=len(got) // 8)
        except AssertionError as e:
            raise AssertionError(f"{cut}: {json.dumps(cfg)}: {e}") from None
        assert eng.cache.live == 0
