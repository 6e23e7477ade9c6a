"""The Lilunex decoder as a layer description.

x = embed[token] * scale. Every sub-layer sits between two norms, x += norm_b(sublayer(norm(x))), and the norm is a
dynamic tanh (tanh(alpha x) * w + b, no statistics). A layer's mixer is "wkv" (token-shifted projections, a matrix state
per head with a decay per key channel that depends on the token, a bonus for the current token), "attention" (biased
projections, queries and keys normalised over the whole projection, partly rotated with linearly scaled frequencies, a
window that also keeps the sequence's first tokens, a sink in the softmax's denominator; optionally the keys and values
another layer cached) or "delta" (gated delta rule with one decay per head). The feed-forward is dense with relu
squared, a mixture of gated experts (softmax router over experts and identity experts, a bias on the choice only,
weights renormalised, a gated shared expert), or absent. Final norm and an untied head. Tensor names: "embed",
"final.norm", "head", and under "l<i>." the layer's "norm1", "norm1b", "mix.*", "norm2", "norm2b", "mlp.*".
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.lilunex import LilunexConfig
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# constants the design fixes
DELTA_UNIT_EPS = 1e-6         # inside the root of the delta rule's unit vectors
ROUTER_SUM_EPS = 1e-20        # added to the sum the chosen experts' scores are divided by


def _mixer_spec(kind: str, m: dict, width: int, eps: float, prefix: str) -> PartSpec:
    if kind == "wkv":
        # (the width of the decay's two-step projection is the weight file's; a configuration may name it, for random weights)
        return PartSpec("wkv", {"hidden": width, "heads": m["heads"], "dim": m["dim"], "eps": eps, "rank": m.get("rank")}, prefix)
    if kind == "delta":
        return PartSpec("gated_delta", {
            "hidden": width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "taps": m["conv"],
            "eps": eps, "decay_per": "head", "low_rank": False, "gate": "silu", "names": {"rate": "a", "gate": "g"}}, prefix)
    rot = m.get("rot") or {"dims": 0, "base": 10000.0}
    mask = m.get("mask") or {}
    factor = float(rot["scaling"]["factor"]) if rot.get("scaling") is not None else 1.0
    return PartSpec("rotary_sink_attention", {
        "hidden": width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "scale": m["scale"],
        "bias": True, "qk_norm_eps": eps, "sink": True, "window": mask.get("size"), "keep_first": mask.get("keep_first") or 0,
        "own_kv": m.get("kv_from") is None,
        "position": PartSpec("rotary", {"rotary_dim": rot["dims"], "theta": rot["base"], "pairing": "half",
                                        "scaling": {"kind": "linear", "factor": factor} if factor != 1.0 else None})}, prefix)


def _feed_forward_spec(f: dict, width: int, prefix: str) -> PartSpec:
    if f["kind"] == "dense":
        return PartSpec("plain_dense", {"hidden": width, "intermediate": f["ff"], "activation": "relu_squared",
                                        "names": {"up": "up", "down": "down"}}, prefix)
    r = f["router"]
    return PartSpec("routed_experts", {
        "hidden": width, "experts": r["experts"], "identity": r.get("identity") or 0, "top": r["top"], "ff": f["expert"]["ff"],
        "score": "softmax", "renormalise": True, "renormalise_eps": ROUTER_SUM_EPS, "scale_input": False, "activation": "swiglu",
        "correction": True, "shared": {"ff": f["shared"]["ff"], "gated": True} if f.get("shared") is not None else None}, prefix)


def lilunex_spec(cfg: LilunexConfig) -> ModelSpec:
    width, eps = cfg.width, cfg.eps
    norm = lambda name, prefix: PartSpec("dynamic_tanh", {"size": width, "weight_name": name}, prefix)
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"mixer_norm": norm("norm1", p), "mixer": _mixer_spec(layer["type"], layer["mixer"], width, eps, p + "mix."),
                 "mixer_post_norm": norm("norm1b", p)}
        if layer["mlp"] is not None:
            parts["feed_forward_norm"] = norm("norm2", p)
            parts["feed_forward"] = _feed_forward_spec(layer["mlp"], width, p + "mlp.")
            parts["feed_forward_post_norm"] = norm("norm2b", p)
        layers.append(LayerSpec(PartSpec("sandwich_norm"), parts))
        schedule.append(ScheduleEntry(i, layer["mixer"].get("kv_from") if layer["type"] == "attention" else None))
    spec = ModelSpec(
        architecture=LilunexConfig.architecture, hidden_size=width, vocab_size=cfg.vocab,
        embedding=PartSpec("table", {"vocab": cfg.vocab, "hidden": width, "name": "embed", "scale": cfg.embedding_scale}),
        layers=layers, schedule=schedule, final_norm=norm("final.norm", ""),
        head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": width, "name": "head", "tied_to": None}),
        max_position=cfg.max_position)
    spec.validate()
    return spec


register_architecture(LilunexConfig.architecture, LilunexConfig, lilunex_spec)
