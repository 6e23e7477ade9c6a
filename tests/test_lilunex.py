"""The Lilunex decoder in the engine against the plain implementation of tests/plain/lilunex_plain.py.

Every test runs on the CPU over the torch stand-ins of the kernels (which checks the parts, the cache manager, the step
function and the scheduler) and, marked gpu, on the real kernels in float32 and bfloat16.
"""
import copy

import pytest
import torch

from serve_b200.cache import CacheManager
from serve_b200.config import ConfigError, PartSpec, build_spec, config_from_dict
from serve_b200.parts import build_part
from tests import helpers
from tests.lilunex_cases import (ATT, BACKENDS, CONFIGS, DELTA, MOE, RANKS, WKV, compare_rows, make_engine, make_weights, plain_logits,
                                 runtime_for, write_model)
from tests.plain import lilunex_plain as P
from tests.test_bapavik import _ctx, _run_part, _tol

LENGTHS = {"a": [1, 5, 23, 49, 75, 130], "o": [3, 40, 90, 17], "q": [2, 9, 31, 64, 101]}
PAGE = {"a": 8, "o": 4, "q": 16}


# ---- configuration and description ----------------------------------------------------------------------------
def test_configuration_is_read_from_the_file_and_describes_every_layer():
    for name, raw in CONFIGS.items():
        cfg = config_from_dict(copy.deepcopy(raw))
        assert type(cfg).__name__ == "LilunexConfig" and cfg.width == raw["width"] and cfg.vocab == raw["vocab"]
        assert cfg.embedding_scale == (raw["embedding"]["scale"] if "embedding" in raw else 1.0)
        spec = build_spec(cfg)
        assert len(spec.layers) == len(raw["layers"]) == len(spec.schedule)
        for i, (layer, ls, entry) in enumerate(zip(raw["layers"], spec.layers, spec.schedule)):
            kinds = {"wkv": "wkv", "delta": "gated_delta", "attention": "rotary_sink_attention"}
            assert ls.parts["mixer"].kind == kinds[layer["type"]]
            assert ("feed_forward" in ls.parts) == (layer["mlp"] is not None)
            assert entry.cache_of == layer["mixer"].get("kv_from")
            if layer["type"] == "attention":
                p = ls.parts["mixer"].params
                assert p["window"] == layer["mixer"]["mask"]["size"] and p["keep_first"] == (layer["mixer"]["mask"].get("keep_first") or 0)
                assert p["own_kv"] == ("kv_from" not in layer["mixer"])
        assert config_from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("breaker", [
    lambda c: c["layers"][0].update(type="conv"),
    lambda c: c["layers"][1]["mixer"].pop("scale"),
    lambda c: c["layers"][1]["mixer"].update(heads=3),
    lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7),
    lambda c: c["layers"][1]["mixer"]["rot"].update(dims=26),
    lambda c: c["layers"][1]["mixer"]["mask"].update(size=0),
    lambda c: c["layers"][3]["mixer"].update(kv_from=3),
    lambda c: c["layers"][3]["mixer"].update(kv_from=2),
    lambda c: c["layers"][3]["mixer"].update(vdim=24),
    lambda c: c["layers"][2]["mixer"].update(kv_heads=3),
    lambda c: c["layers"][0]["mlp"]["router"].update(top=9),
    lambda c: c["layers"][0]["mlp"].update(kind="sparse"),
    lambda c: c["norm"].update(eps=0.0),
    lambda c: c.pop("vocab"),
])
def test_configuration_refuses_what_it_cannot_run(breaker):
    raw = copy.deepcopy(CONFIGS["a"])
    breaker(raw)
    with pytest.raises(ConfigError):
        config_from_dict(raw)


def test_the_owner_of_shared_keys_keeps_what_its_readers_look_at():
    """Layer 3 of "a" reads layer 1's pages through a longer window and more kept tokens: the pages' group has both."""
    from serve_b200.engine.runtime import Runtime
    from serve_b200.models import DecoderModel
    from tests.emu_kernels import EmuKernels

    spec = build_spec(config_from_dict(copy.deepcopy(CONFIGS["a"])))
    needs = DecoderModel(spec, Runtime(EmuKernels("cpu"), "cpu", torch.float32)).cache_needs()
    assert needs[3] is None and needs[1].window == 33 and needs[1].keep_first == 5
    mgr = CacheManager(needs, [e.cache_of for e in spec.schedule], 4, 64, 2, 256, device="cpu", kv_dtype=torch.float32)
    mgr.open("r")
    mgr.reserve([("r", 100)])
    mgr.commit("r", 100)
    g = mgr.groups[mgr.views()[1].group]
    row = g.table[mgr.slot("r")]
    assert all(row[b] >= 0 for b in (0, 1)) and all(row[b] < 0 for b in range(2, (100 - 33 + 1) // 4))
    assert all(row[b] >= 0 for b in range((100 - 33 + 1) // 4, 25))
    assert mgr.views()[3].k is mgr.views()[1].k and not mgr.views()[3].writes


# ---- whole models ---------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """{config name: {dtype: (weights, requests, plain logits, model folder)}}."""
    out = {}
    for name in LENGTHS:
        cfg = CONFIGS[name]
        reqs = {f"r{i}": helpers.random_tokens(cfg["vocab"], n, seed=20 + i) for i, n in enumerate(LENGTHS[name])}
        w = make_weights(cfg, 100 + len(name), RANKS[name])
        plain = {rid: plain_logits(w, cfg, toks) for rid, toks in reqs.items()}
        out[name] = {dt: (w, reqs, plain, write_model(str(tmp_path_factory.mktemp(f"{name}-{dt}")), cfg, w, getattr(torch, dt)))
                     for dt in ("float32", "bfloat16")}
    return out


def test_plain_layers_feed_one_another(models):
    """The oracle's own premise: every layer changes the residual stream, and the last positions depend on the first token."""
    for name in LENGTHS:
        w, reqs, plain, _ = models[name]["float32"]
        toks = reqs["r2"]
        layers = []
        plain_logits(w, CONFIGS[name], toks, layers)
        for a, b in zip(layers, layers[1:]):
            assert float((a - b).abs().max()) > 1e-2
        other = [(toks[0] + 1) % CONFIGS[name]["vocab"]] + toks[1:]
        assert float((plain_logits(w, CONFIGS[name], other)[-1] - plain[f"r2"][-1]).abs().max()) > 1e-4


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
    having been written shows; a slot's states must start from zero whoever had the slot before."""
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
    """Two requests decoded one token at a time for 120 steps after short prompts (from CUDA graphs on the GPU): the window
    of 64 passes over decoded tokens, pages are crossed and given back many times, the kept first tokens stay."""
    cfg = CONFIGS["q"]
    w, _, _, folder = models["q"][backend[1]]
    seqs = {f"d{i}": helpers.random_tokens(cfg["vocab"], 140 - 9 * i, seed=60 + i) for i in range(2)}
    plain = {rid: plain_logits(w, cfg, toks) for rid, toks in seqs.items()}
    eng = make_engine(folder, backend, 16, num_pages=16, graphs=True)
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
    assert max(g.pool.high_water for g in eng.cache.groups) <= 2 * (64 // 16 + 2 + 2)      # pages behind the window came back


@pytest.mark.parametrize("backend", BACKENDS)
def test_greedy_generation_through_the_scheduler(models, backend):
    """generate(): the engine's own entry point, scheduler and sampler. Every generated token must be (within the
    tolerance) the best one of the plain model given the tokens before it."""
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
F64 = lambda w: {k: v.double() for k, v in w.items() if v.dtype.is_floating_point}


def _single(kind, mixer=None, mlp=None, width=64):
    """A one-layer configuration around the mechanism under test."""
    return {"architecture": "Lilunex", "width": width, "vocab": 50, "norm": {"eps": 1e-5}, "embedding": {"scale": 4.0},
            "layers": [{"type": kind, "mixer": mixer, "mlp": mlp}]}


def _mixer_alone(backend, cfg, cuts, seed=5, x=None, tweak=None, page=8, loose=1.0, rank=8):
    from serve_b200.models.lilunex import _mixer_spec

    layer = cfg["layers"][0]
    w = make_weights(cfg, seed, rank)
    if tweak is not None:
        tweak(w, "l0.mix.")
    if x is None:
        x = torch.randn(sum(cuts), cfg["width"], generator=torch.Generator().manual_seed(seed + 1))
    x = x.bfloat16().float()
    spec = _mixer_spec(layer["type"], layer["mixer"], cfg["width"], cfg["norm"]["eps"], "l0.mix.")
    got = _run_part(backend, "mixer", spec, w, x, cuts, page=page)
    w64, m, eps = F64(w), layer["mixer"], cfg["norm"]["eps"]
    if layer["type"] == "attention":
        want = P.attention_mixer(x.double(), w64, "l0.mix.", m, eps, *P.attention_keys_values(x.double(), w64, "l0.mix.", m, eps)).float()
    else:
        want = {"wkv": P.wkv_mixer, "delta": P.delta_mixer}[layer["type"]](x.double(), w64, "l0.mix.", m, eps).float()
    torch.testing.assert_close(got, want, atol=_tol(backend, want) * loose, rtol=0)
    return got, want, w


WKVS = [WKV(2, 16), WKV(5, 12), WKV(1, 32), WKV(3, 64)]
DELTAS = [DELTA(4, 2, 16, 24, 4), DELTA(3, 3, 12, 20, 3), DELTA(6, 2, 8, 8, 2), DELTA(2, 1, 64, 32, 4)]
ATTS = [ATT(4, 2, 24, 16, 0.2, 20, 3, 10000.0, 16, 2.0), ATT(6, 1, 20, 12, 0.3, 7, None, 3000.0, 10, None),
        ATT(6, 3, 8, 8, 0.35, 64, 17, 100.0, 8, 8.0), ATT(2, 2, 16, 40, 0.25, 9, 9, 500.0, 0, None),
        ATT(3, 1, 32, 32, 0.18, 1, 2, 7000.0, 32, 0.5),
        {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.3}]     # no mask and no rotation in the file


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("cuts", CUTS, ids=["whole", "portions", "tokens"])
@pytest.mark.parametrize("which", range(len(WKVS)))
def test_wkv_alone(backend, cuts, which):
    _mixer_alone(backend, _single("wkv", WKVS[which], width=(64, 100, 48, 72)[which]), cuts, rank=(8, 5, 12, 16)[which], loose=2.0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("cuts", CUTS, ids=["whole", "portions", "tokens"])
@pytest.mark.parametrize("which", range(len(DELTAS)))
def test_gated_delta_alone(backend, cuts, which):
    _mixer_alone(backend, _single("delta", DELTAS[which], width=(64, 100, 48, 72)[which]), cuts, loose=2.0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("cuts", CUTS, ids=["whole", "portions", "tokens"])
@pytest.mark.parametrize("which", range(len(ATTS)))
def test_attention_alone(backend, cuts, which):
    """Also: no rotation at all, a window of one key (the query's own) with two kept tokens, value heads wider than the
    keys', a window as long as the kept tokens, a mixer whose file names neither a mask nor a rotation (every earlier
    position is seen, no position signal)."""
    _mixer_alone(backend, _single("attention", ATTS[which], width=(64, 100, 48, 40, 72, 56)[which]), cuts)


def test_the_first_tokens_of_a_sequence_start_from_zeros():
    """The oracle's premise for the first tokens: the token before the first is zeros (token shift, convolution) and the
    state is zero, so the first token's output is a function of that token alone."""
    for kind, m in (("wkv", WKVS[0]), ("delta", DELTAS[0])):
        cfg = _single(kind, m)
        w = F64(make_weights(cfg, 3))
        x = torch.randn(6, 64, generator=torch.Generator().manual_seed(4)).double()
        fn = {"wkv": P.wkv_mixer, "delta": P.delta_mixer}[kind]
        full = fn(x, w, "l0.mix.", m, 1e-5)
        torch.testing.assert_close(fn(x[:1], w, "l0.mix.", m, 1e-5), full[:1])
        assert float((fn(x[1:], w, "l0.mix.", m, 1e-5)[0] - full[1]).abs().max()) > 1e-3


@pytest.mark.parametrize("backend", BACKENDS)
def test_states_of_a_slot_are_cleared_for_the_next_request(backend):
    """A recurrent mixer over a sequence, after another sequence ran in the same slot and was closed (``_run_part`` does
    that with five tokens; here the earlier one is long, so that its state and its last input are far from zero)."""
    from serve_b200.models.lilunex import _mixer_spec

    for kind, m in (("wkv", WKVS[0]), ("delta", DELTAS[0])):
        cfg = _single(kind, m)
        w = make_weights(cfg, 8)
        rt, dev = runtime_for(backend)
        part = build_part("mixer", _mixer_spec(kind, m, 64, 1e-5, "l0.mix."), rt)
        part.load({d.name: w[d.name].to(dev).to(rt.act_dtype if w[d.name].dim() > 1 else torch.float32) for d in part.tensor_decls()})
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
        want = {"wkv": P.wkv_mixer, "delta": P.delta_mixer}[kind](x.double(), F64(w), "l0.mix.", m, 1e-5).float()
        torch.testing.assert_close(outs[1], want, atol=2 * _tol(backend, want), rtol=0)


def _attention_pair(backend, owner, reader, cuts, seed=21, width=64, page=8, x=None, tweak=None):
    """An attention layer and a second one that reads the first one's pages through its own mask, over one sequence."""
    from serve_b200.models.lilunex import _mixer_spec

    cfg = {"architecture": "Lilunex", "width": width, "vocab": 50, "norm": {"eps": 1e-5},
           "layers": [{"type": "attention", "mixer": owner, "mlp": None}, {"type": "attention", "mixer": reader, "mlp": None}]}
    w = make_weights(cfg, seed)
    if tweak is not None:
        tweak(w)
    rt, dev = runtime_for(backend)
    parts = [build_part("mixer", _mixer_spec("attention", m, width, 1e-5, f"l{i}.mix."), rt) for i, m in enumerate((owner, reader))]
    for part in parts:
        part.load({d.name: w[d.name].to(dev).to(rt.act_dtype if w[d.name].dim() > 1 else torch.float32) for d in part.tensor_decls()})
    need = parts[0].cache_need().covering(parts[1].cache_need())
    mgr = CacheManager([need, None], [None, 0], page, 128, 1, 4096, device=dev, kv_dtype=rt.act_dtype)
    views = mgr.views()
    if x is None:
        x = torch.randn(sum(cuts), width, generator=torch.Generator().manual_seed(seed + 1))
    x = x.bfloat16().float()
    y = (x.flip(1) * 0.7).bfloat16().float()                                            # the reader's input is another one
    xs = [x.to(dev).to(rt.act_dtype), y.to(dev).to(rt.act_dtype)]
    outs, at = [], 0
    with torch.inference_mode():
        mgr.open("r")
        for n in cuts:
            mgr.reserve([("r", at + n)])
            ctx = _ctx(rt, dev, [n], [at], [mgr.slot("r")], mgr, ["r"])
            parts[0].forward(xs[0][at: at + n], ctx, views[0])
            outs.append(parts[1].forward(xs[1][at: at + n], ctx, views[1]).float().cpu())
            mgr.commit("r", at + n)
            at += n
    rt.kernels.check_errors()
    w64 = F64(w)
    k, v = P.attention_keys_values(x.double(), w64, "l0.mix.", owner, 1e-5)
    want = P.attention_mixer(y.double(), w64, "l1.mix.", reader, 1e-5, k, v).float()
    got = torch.cat(outs)
    torch.testing.assert_close(got, want, atol=_tol(backend, want), rtol=0)
    return got, want


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("cuts", [[90], [40, 1, 1, 2, 25, 1, 20], [1] * 90], ids=["whole", "portions", "tokens"])
@pytest.mark.parametrize("masks", [((20, 3), (33, 5)), ((33, 5), (20, 3)), ((7, 0), (50, 9)), ((12, 2), (12, 2))])
def test_attention_over_another_layers_keys(backend, cuts, masks):
    """The reader's window is longer or shorter than the owner's, with more or fewer kept tokens: pages are given back
    only when neither looks at them any more."""
    (s0, k0), (s1, k1) = masks
    owner = ATT(4, 2, 24, 16, 0.2, s0, k0, 10000.0, 16, 2.0)
    reader = ATT(4, 2, 24, 16, 0.3, s1, k1, 10000.0, 16, 2.0, kv_from=0)
    _attention_pair(backend, owner, reader, cuts)


# ---- keys far away, at page borders, at the window's and the kept tokens' edges -----------------------------------
def _stand_out(width, n, key, query, seed=4):
    """Inputs of which token ``key`` is large and token ``query`` is minus three times it, all others small."""
    x = torch.randn(n, width, generator=torch.Generator().manual_seed(seed)) * 0.3
    x[key] = torch.randn(width, generator=torch.Generator().manual_seed(seed + 1)) * 1.5
    if query != key:
        x[query] = -3.0 * x[key]
    return x


def _pointing(m):
    """Weights with which a query made from minus a key's token points along that key: W_q = -W_k per group, biases off, the
    query norm three times the key norm, a low sink. The rotation is slow (large base, few rotated elements), so it turns
    the pair by little over hundreds of positions."""
    rep = m["heads"] // m["kv_heads"]

    def tweak(w, prefix):
        w[prefix + "q"] = -w[prefix + "k"].view(m["kv_heads"], m["dim"], -1).repeat_interleave(rep, 0).reshape(m["heads"] * m["dim"], -1).clone()
        w[prefix + "q.norm"] = 3.0 * w[prefix + "k.norm"].view(m["kv_heads"], m["dim"]).repeat_interleave(rep, 0).reshape(-1).clone()
        w[prefix + "q.b"] = w[prefix + "q.b"] * 0
        w[prefix + "k.b"] = w[prefix + "k.b"] * 0
        w[prefix + "sink"] = w[prefix + "sink"] * 0 - 2.0
    return tweak


def _sees(m, query, key):
    return P.visible(query, key, m["mask"]["size"], m["mask"].get("keep_first") or 0)


def _edge_case(backend, m, key, query, cuts, page=8):
    cfg = _single("attention", m)
    x = _stand_out(64, sum(cuts), key, query)
    # (the query token is minus three times the key token, so a few outputs are large: one rounding more of them counts)
    got, want, w = _mixer_alone(backend, cfg, cuts, seed=11, x=x, tweak=_pointing(m), page=page, loose=1.5)
    # the premise: where the mask lets the query see the key, the key carries the output (without it the output is another
    # one); where it does not, the key changes nothing
    x2 = x.bfloat16().float().clone()
    x2[key] = 0.0
    w64 = F64(w)
    other = P.attention_mixer(x2.double(), w64, "l0.mix.", m, 1e-5, *P.attention_keys_values(x2.double(), w64, "l0.mix.", m, 1e-5)).float()
    moved = float((other[query] - want[query]).abs().max())
    if key != query:
        assert (moved > 20 * _tol(backend, want)) == _sees(m, query, key), (key, query, moved)


SLOW = dict(base=1e6, dims=8, factor=4.0)
# a window of 37 keys and 5 kept tokens over pages of 8: (key, query) pairs just inside and just outside the window, at page
# borders (256 | 255, 263 | 264), among the kept tokens and just past them, the first key of all, and the query's own
EDGES = [(263, 299), (262, 299), (256, 292), (255, 292), (264, 300 - 1), (0, 299), (4, 299), (5, 299), (4, 41), (5, 41), (5, 42), (7, 8),
         (8, 44), (8, 45), (299, 299), (63, 64), (1, 38)]
EDGE_CUTS = [[300], [270] + [1] * 30, [100, 2, 150, 3, 45], [36, 2, 2, 2, 258]]


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("key,query", EDGES)
@pytest.mark.parametrize("cuts", EDGE_CUTS, ids=["prompt", "decoded", "portions", "early_cuts"])
def test_attention_sees_exactly_the_window_and_the_kept_tokens(backend, key, query, cuts):
    m = ATT(4, 2, 24, 16, 0.2, 37, 5, SLOW["base"], SLOW["dims"], SLOW["factor"])
    _edge_case(backend, m, key, query, cuts)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("size,keep,key,query", [(64, 17, 16, 299), (64, 17, 17, 299), (64, 17, 236, 299), (64, 17, 235, 299),
                                                 (128, 0, 0, 127), (128, 0, 0, 128), (200, 70, 69, 299), (200, 70, 70, 299),
                                                 (16, 16, 15, 200), (16, 16, 16, 200), (3, 1, 0, 250), (3, 1, 1, 250), (3, 1, 248, 250)])
@pytest.mark.parametrize("cuts", [[300], [240] + [1] * 60, [130, 2, 100, 3, 65]], ids=["prompt", "decoded", "portions"])
def test_other_windows_and_kept_counts(backend, size, keep, key, query, cuts):
    """Kept tokens that fill more than one page and exactly one, none at all, a window of a page's size and of several
    pages, and a tiny one: pages of 16."""
    m = ATT(4, 4, 16, 16, 0.25, size, keep, SLOW["base"], SLOW["dims"], SLOW["factor"])
    _edge_case(backend, m, key, query, cuts, page=16)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("sink", [-30.0, 0.0, 6.0, 40.0])
def test_the_sink_takes_its_share_once(backend, sink):
    """A sink far below the scores changes nothing, one far above them takes all the weight (the output goes to the output
    projection's bias); decoded over many keys (where the kernels split the keys over blocks and merge) it counts once."""
    m = ATT(4, 2, 24, 16, 0.2, 350, 3, 10000.0, 16, 2.0)
    cfg = _single("attention", m)

    def tweak(w, prefix):
        w[prefix + "sink"] = torch.full_like(w[prefix + "sink"], sink)

    for cuts in ([400], [399, 1], [200] + [1] * 200):
        got, want, w = _mixer_alone(backend, cfg, cuts, seed=13, tweak=tweak)
    if sink >= 40.0:
        assert float((want - w["l0.mix.o.b"]).abs().max()) < 1e-6
    if sink <= -30.0:
        w["l0.mix.sink"] = torch.full_like(w["l0.mix.sink"], -1e4)
        x = torch.randn(400, 64, generator=torch.Generator().manual_seed(14)).bfloat16().double()
        w64 = F64(w)
        none = P.attention_mixer(x, w64, "l0.mix.", m, 1e-5, *P.attention_keys_values(x, w64, "l0.mix.", m, 1e-5)).float()
        torch.testing.assert_close(want, none, atol=1e-5 * float(none.abs().max()), rtol=0)


@pytest.mark.parametrize("backend", BACKENDS)
def test_rotation_far_from_the_start(backend):
    """Fast rotation (small base, all of a head rotated, frequencies scaled up by a factor below one) at positions in the
    thousands: the angle must be computed from the true position in 32 bits, in prompts and in decoding."""
    m = ATT(2, 1, 16, 16, 0.25, 48, 2, 50.0, 16, 0.5)
    cfg = _single("attention", m)
    n = 2100
    _mixer_alone(backend, cfg, [2048, 30] + [1] * 22, seed=17, page=64, x=torch.randn(n, 64, generator=torch.Generator().manual_seed(18)), loose=4.0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("kind", ["wkv", "delta"])
def test_a_state_carries_the_first_token_over_hundreds(backend, kind):
    """Decays close to one: what the first token wrote into the state still shows 300 tokens later, through every cut."""
    m = WKVS[0] if kind == "wkv" else DELTAS[0]
    cfg = _single(kind, m)

    def tweak(w, prefix):
        if kind == "wkv":
            w[prefix + "w0"] = torch.full_like(w[prefix + "w0"], -7.0)
            w[prefix + "w2"] = w[prefix + "w2"] * 0.1
        else:
            w[prefix + "A_log"] = torch.full_like(w[prefix + "A_log"], -7.0)

    x = torch.randn(300, 64, generator=torch.Generator().manual_seed(30)) * 0.5
    x[0] = x[0] * 6.0
    for cuts in ([300], [100, 2, 150, 3, 45], [260] + [1] * 40):
        got, want, w = _mixer_alone(backend, cfg, cuts, seed=29, x=x, tweak=tweak, loose=4.0)
    x2 = x.bfloat16().double().clone()
    x2[0] = 0.0
    other = {"wkv": P.wkv_mixer, "delta": P.delta_mixer}[kind](x2, F64(w), "l0.mix.", m, 1e-5).float()
    assert float((other[299] - want[299]).abs().max()) > 10 * _tol(("emu", "float32"), want)


# ---- feed-forwards, norm, token shift ------------------------------------------------------------------------
@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("width,ff", [(64, 96), (100, 70), (48, 64), (512, 1024)])
def test_dense_feed_forward_alone(backend, width, ff):
    from serve_b200.models.lilunex import _feed_forward_spec

    cfg = _single("wkv", WKVS[0], DENSE_FF(ff), width)
    w = make_weights(cfg, 21)
    # (few rows, some, and at the widest size thousands: in bfloat16 on the GPU the few-rows product, the library product
    # with the activation kernel, and the tensor-memory product, the first and the last with the activation in their epilogue)
    for rows in (70, 5, 300) + ((2048,) if width == 512 and backend[0] == "cuda" else ()):
        x = torch.randn(rows, width, generator=torch.Generator().manual_seed(22)).bfloat16().float()
        want = P.dense_ff(x.double(), F64(w), "l0.mlp.").float()
        assert float((x.double() @ w["l0.mlp.up"].double().T < 0).double().mean()) > 0.3      # the relu really cuts
        got = _run_part(backend, "feed_forward", _feed_forward_spec(cfg["layers"][0]["mlp"], width, "l0.mlp."), w, x, [rows], pages=64)
        torch.testing.assert_close(got, want, atol=_tol(backend, want), rtol=0)


DENSE_FF = lambda ff: {"kind": "dense", "ff": ff}
MOES = [(64, MOE(6, 2, 2, 32, shared=48)), (100, MOE(5, 3, 3, 22, shared=30)), (48, MOE(7, 1, 2, 16, shared=16)), (64, MOE(4, 0, 1, 48)),
        (100, MOE(3, 1, 4, 30)), (128, MOE(8, 4, 3, 64, shared=96)), (64, MOE(2, 6, 2, 32))]


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("which", range(len(MOES)))
def test_experts_alone(backend, which):
    """Routed experts with identity outputs, a choice bias and a gated shared expert, one token at a time and many: also
    every output chosen at once, one choice a token, no identity outputs, more identity outputs than experts."""
    from serve_b200.models.lilunex import _feed_forward_spec

    width, f = MOES[which]
    cfg = _single("wkv", WKVS[0], f, width)
    w = make_weights(cfg, 23)
    x = torch.randn(70, width, generator=torch.Generator().manual_seed(25)).bfloat16().float()
    w64 = F64(w)
    want = P.moe_ff(x.double(), w64, "l0.mlp.", f).float()
    chosen, weights = P.router_choice(x.double(), w64, "l0.mlp.", f)
    n_out = f["router"]["experts"] + f["router"]["identity"]
    if f["router"]["top"] < n_out:
        # premises: the bias changes some choices, identity outputs are chosen (where there are any), and no choice is a close call
        s = torch.softmax(x.double() @ w64["l0.mlp.router"].T, -1)
        unbiased = torch.topk(s, f["router"]["top"], dim=-1).indices
        assert (unbiased.sort(-1).values != chosen.sort(-1).values).any()
        ranked = (s + w64["l0.mlp.correction"]).sort(-1, descending=True).values
        assert float((ranked[:, f["router"]["top"] - 1] - ranked[:, f["router"]["top"]]).min()) > 1e-5
    if f["router"]["identity"]:
        assert (chosen >= f["router"]["experts"]).any()
    spec = _feed_forward_spec(f, width, "l0.mlp.")
    for cuts in ([70], [3, 1, 40, 26], [1] * 70):
        got = _run_part(backend, "feed_forward", spec, w, x, cuts)
        torch.testing.assert_close(got, want, atol=_tol(backend, want) * 2, rtol=0)


@pytest.mark.parametrize("backend", BACKENDS)
def test_the_router_weights_use_the_scores_without_the_bias(backend):
    """A large bias on one expert makes every token choose it, while its weight stays its small score: with the bias in the
    weights the output would be another one."""
    from serve_b200.models.lilunex import _feed_forward_spec

    f = MOE(5, 1, 2, 32)
    cfg = _single("wkv", WKVS[0], f, 64)
    w = make_weights(cfg, 27)
    w["l0.mlp.correction"] = torch.tensor([0.0, 0.0, 0.0, 5.0, 0.0, 0.0])
    x = torch.randn(33, 64, generator=torch.Generator().manual_seed(28)).bfloat16().float()
    w64 = F64(w)
    chosen, weights = P.router_choice(x.double(), w64, "l0.mlp.", f)
    assert bool((chosen == 3).any(-1).all()) and float(weights[chosen == 3].mean()) < 0.4
    want = P.moe_ff(x.double(), w64, "l0.mlp.", f).float()
    got = _run_part(backend, "feed_forward", _feed_forward_spec(f, 64, "l0.mlp."), w, x, [33])
    torch.testing.assert_close(got, want, atol=_tol(backend, want) * 2, rtol=0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("width", [48, 100, 512, 1030])
def test_dynamic_tanh_alone_and_behind_another(backend, width):
    """The norm on the residual stream, with a plain delta, with a delta that still has to pass a norm of its own (applied
    in the same kernel), for picked rows, and on activations that are not the residual stream."""
    from serve_b200.parts.base import DeferredNorm

    rt, dev = runtime_for(backend)
    g = torch.Generator().manual_seed(width)
    w = {}
    for n in ("t.a", "t.b"):
        w[n] = (1.0 + 0.3 * torch.randn(width, generator=g)).bfloat16().float()
        w[n + ".b"] = (0.2 * torch.randn(width, generator=g)).bfloat16().float()
        w[n + ".alpha"] = torch.tensor(0.4 if n == "t.a" else 1.3).bfloat16().float()
    norms = {}
    for n in ("a", "b"):
        norms[n] = build_part("norm", PartSpec("dynamic_tanh", {"size": width, "weight_name": n}, "t."), rt)
        norms[n].load({k: v.to(dev) for k, v in w.items()})
    w64 = F64(w)
    x = torch.randn(37, width, generator=g) * 2.0
    delta = torch.randn(37, width, generator=g).to(rt.act_dtype)
    # a plain delta
    xs = x.clone().to(dev)
    got = norms["a"].forward(xs, delta.to(dev), None).float().cpu()
    want_x = x + delta.float()
    torch.testing.assert_close(xs.cpu(), want_x, atol=1e-6, rtol=0)
    want = P.dyn_tanh(want_x.double(), w64, "t.a").float()
    torch.testing.assert_close(got, want, atol=_tol(backend, want) * 2, rtol=0)
    # a delta behind norm b, as activations and as float sums
    for d in (delta, delta.float() * 1.5):
        xs = x.clone().to(dev)
        got = norms["a"].forward(xs, DeferredNorm(d.to(dev), norms["b"]), None).float().cpu()
        want_x = (x.double() + P.dyn_tanh(d.double(), w64, "t.b")).float()
        torch.testing.assert_close(xs.cpu(), want_x, atol=2e-6, rtol=0)
        want = P.dyn_tanh(want_x.double(), w64, "t.a").float()
        torch.testing.assert_close(got, want, atol=_tol(backend, want) * 2, rtol=0)
    # picked rows: x stays as it is
    rows = torch.tensor([5, 0, 36], dtype=torch.int32, device=dev)
    xs = x.clone().to(dev)
    got = norms["a"].forward_rows(xs, DeferredNorm(delta.to(dev), norms["b"]), rows, None).float().cpu()
    torch.testing.assert_close(xs.cpu(), x, atol=0, rtol=0)
    want = P.dyn_tanh(x.double() + P.dyn_tanh(delta.double(), w64, "t.b"), w64, "t.a").float()[[5, 0, 36]]
    torch.testing.assert_close(got, want, atol=_tol(backend, want) * 2, rtol=0)
    # no delta at all, and the norm of activations
    got = norms["a"].forward(x.clone().to(dev), None, None).float().cpu()
    torch.testing.assert_close(got, P.dyn_tanh(x.double(), w64, "t.a").float(), atol=_tol(backend, want) * 2, rtol=0)
    got = norms["b"].apply(delta.to(dev)).cpu()
    torch.testing.assert_close(got, P.dyn_tanh(delta.double(), w64, "t.b").float(), atol=1e-5, rtol=0)


@pytest.mark.parametrize("backend", BACKENDS)
def test_token_shift_alone(backend):
    rt, dev = runtime_for(backend)
    width = 100
    g = torch.Generator().manual_seed(3)
    mu = {f"s.mu.{c}": torch.rand(width, generator=g).bfloat16().float() for c in "abc"}
    part = build_part("filter", PartSpec("token_shift", {"channels": width, "mixes": ["mu.a", "mu.b", "mu.c"]}, "s."), rt)
    part.load({k: v.to(dev) for k, v in mu.items()})
    x = torch.randn(41, width, generator=g).bfloat16().float()
    prev = torch.cat([torch.zeros(1, width), x[:-1]])
    want = torch.stack([x + (prev - x) * mu[f"s.mu.{c}"] for c in "abc"])
    for cuts in ([41], [1] * 41, [7, 1, 2, 30, 1]):
        mgr = CacheManager([part.cache_need()], [None], 8, 8, 2, 64, device=dev, kv_dtype=rt.act_dtype)
        view = mgr.views()[0]
        mgr.open("x")
        mgr.open("r")
        outs, at = [], 0
        with torch.inference_mode():
            for n in cuts:
                ctx = _ctx(rt, dev, [n], [at], [mgr.slot("r")])
                outs.append(part.forward(x[at: at + n].to(dev).to(rt.act_dtype), ctx, view).float().cpu())
                at += n
        torch.testing.assert_close(torch.cat(outs, 1), want, atol=_tol(backend, want), rtol=0)


# ---- sizes of a real layer, and the programs a user starts ------------------------------------------------------
@pytest.mark.parametrize("backend", BACKENDS[1:])
@pytest.mark.parametrize("index", [0, 1, 2], ids=["attention", "wkv", "delta"])
@pytest.mark.parametrize("cuts", [[420], [130, 1, 1, 270, 18]], ids=["whole", "portions"])
def test_mixers_at_the_sizes_of_a_real_layer(backend, index, cuts):
    """Each mixer alone at heads of 64 and 128 over 420 tokens, whole and cut with single tokens in the middle."""
    layer = CONFIGS["wide"]["layers"][index]
    _mixer_alone(backend, _single(layer["type"], layer["mixer"], width=512), cuts, seed=31, page=64, rank=32, loose=2.0)


@pytest.mark.parametrize("backend", BACKENDS[1:])
def test_a_model_at_the_sizes_of_a_real_layer(backend, tmp_path):
    cfg = CONFIGS["wide"]
    w = make_weights(cfg, 41, RANKS["wide"])
    folder = write_model(str(tmp_path / "wide"), cfg, w, getattr(torch, backend[1]))
    reqs = {f"r{i}": helpers.random_tokens(cfg["vocab"], n, seed=50 + i) for i, n in enumerate([400, 37, 170])}
    tail = {rid: min(45, len(toks)) for rid, toks in reqs.items()}
    plain = {rid: plain_logits(w, cfg, toks)[-tail[rid]:] for rid, toks in reqs.items()}
    eng = make_engine(folder, backend, 64, num_pages=12, graphs=True, budget=512)
    steps = helpers.trace_mixed(reqs, live=3, seed=5, decode_tail=20, budget=256)
    with torch.inference_mode():
        got = helpers.replay(eng, steps)
    eng.kernels.check_errors()
    got = {(rid, pos - (len(reqs[rid]) - tail[rid])): row for (rid, pos), row in got.items() if pos >= len(reqs[rid]) - tail[rid]}
    assert len(got) > 60
    compare_rows(got, plain, backend)


@pytest.mark.gpu
def test_trace_run_and_command_line_programs(models, tmp_path):
    """bin/trace_run and `python -m serve_b200.run` as a user starts them, on a model folder of this design: the class is
    chosen by config.json; four slots and a pool smaller than the requests' total, so slots and pages come again."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype in ("float32", "bfloat16"):
        w, reqs, plain, folder = models["a"][dtype]
        steps = helpers.trace_mixed(reqs, live=4, seed=9)
        need = helpers.tokens_needed(steps, 64)
        out_dir = tmp_path / f"out-{dtype}"
        proc = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", str(out_dir),
                               "--max-tokens", str(need)], input="\n".join(json.dumps(s) for s in steps) + "\n",
                              capture_output=True, text=True, timeout=900)
        assert proc.returncode == 0, proc.stderr[-3000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
        got, at = {}, {}
        for s in steps:
            n_want = sum(len(e["want"]) for e in s["entries"])
            if not n_want:
                continue
            arr = np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4").reshape(n_want, CONFIGS["a"]["vocab"])
            i = 0
            for e in s["entries"]:
                base = at.get(e["id"], 0)
                for wi in e["want"]:
                    got[(e["id"], base + wi)] = torch.from_numpy(arr[i].copy())
                    i += 1
            for e in s["entries"]:
                at[e["id"]] = at.get(e["id"], 0) + len(e["tokens"])
        compare_rows(got, plain, ("cuda", dtype))
    w, reqs, plain, folder = models["a"]["float32"]
    prompt = reqs["r2"]
    out = subprocess.run([sys.executable, "-m", "serve_b200.run", "--model", folder, "--dtype", "float32", "--page-size", "8", "--num-pages",
                          "16", "--max-context", "64", "--max-slots", "2", "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "4"],
                         cwd=root, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    new = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])["generated_tokens"]
    logits = plain_logits(w, CONFIGS["a"], prompt + new)
    assert all(int(logits[len(prompt) - 1 + i].argmax()) == t for i, t in enumerate(new))


ONE_KIND = {
    "recurrent": {"architecture": "Lilunex", "width": 64, "vocab": 90, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0}, "layers": [
        {"type": "wkv", "mixer": WKV(2, 16), "mlp": None}, {"type": "delta", "mixer": DELTA(2, 1, 16, 16, 3), "mlp": None}]},
    "attention": {"architecture": "Lilunex", "width": 64, "vocab": 90, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0}, "layers": [
        {"type": "attention", "mixer": ATT(2, 1, 16, 16, 0.25, 300, 0, 1000.0, 16, 1.0), "mlp": {"kind": "dense", "ff": 64}},
        {"type": "attention", "mixer": ATT(2, 1, 16, 16, 0.25, 5, 1, 1000.0, 16, 1.0, kv_from=0), "mlp": None},
        {"type": "attention", "mixer": ATT(4, 4, 8, 8, 0.3, 9, 2, 1000.0, 4, 3.0), "mlp": None},
        {"type": "attention", "mixer": ATT(2, 1, 16, 16, 0.25, 11, 20, 1000.0, 16, 1.0, kv_from=0), "mlp": MOE(2, 0, 2, 16)}]},
}


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("kind", sorted(ONE_KIND))
def test_models_of_one_kind_of_layer(backend, kind, tmp_path):
    """No cached keys at all (no page group, only states), and nothing but attention (no state; two layers read the
    first one's keys through windows of their own, one of them with more kept tokens than its window is long)."""
    cfg = ONE_KIND[kind]
    w = make_weights(cfg, 7)
    folder = write_model(str(tmp_path / kind), cfg, w, getattr(torch, backend[1]))
    reqs = {f"r{i}": helpers.random_tokens(cfg["vocab"], n, seed=i) for i, n in enumerate([70, 3, 41])}
    plain = {rid: plain_logits(w, cfg, t) for rid, t in reqs.items()}
    eng = make_engine(folder, backend, 8, num_pages=24, max_slots=2)
    assert len(eng.cache.groups) == (0 if kind == "recurrent" else 2)
    with torch.inference_mode():
        got = helpers.replay(eng, helpers.trace_mixed(reqs, live=2, seed=3))
    eng.kernels.check_errors()
    compare_rows(got, plain, backend)
    assert eng.cache.live == 0
