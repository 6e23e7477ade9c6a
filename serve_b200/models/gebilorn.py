"""The Gebilorn decoder as a layer description.

x = embed[token] * scale + pairs[(previous token * a + token * b) mod buckets] (the table's last row for a sequence's
first token). A layer has one norm, rms with a weight stored as its distance from one, and both sub-layers read its
output: x += mixer(h) + ff(h). A layer's mixer is "attention" (grouped queries, a part of every head rotated with
frequencies scaled band by band, queries and keys divided by their own root mean square per head after the rotation, a
window that also keeps the sequence's first tokens, a sink in the softmax's denominator, an element-wise sigmoid gate on
the heads' outputs), "parallel" (biased projections through short convolutions, a plain window, a sink and one sigmoid
gate per head, beside a matrix state per head with a decay per key channel; summed with fixed scales) or
"latent_attention" (queries through a normalised low-rank step, keys and values read out of one normalised low-rank
vector per token plus one rotated key part shared by all heads). The feed-forward is dense and gated with the tanh form
of gelu, a mixture of silu-gated experts (softmax router, weights = chosen scores times a constant, a gated shared
expert), or absent. Final norm, the embedding table as head, capped logits. Tensor names: "embed", "bigram",
"final.norm", and under "l<i>." the layer's "norm1", "mix.*", "mlp.*".
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.gebilorn import GebilornConfig
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _rotary(rot, dims=None) -> PartSpec:
    if not rot or not (dims if dims is not None else rot["dims"]):
        return PartSpec("none")
    sc = rot.get("scaling")
    scaling = None if not sc else {"factor": sc["factor"], "low_freq_factor": sc["low"], "high_freq_factor": sc["high"],
                                   "original_max_position_embeddings": sc["original"]}
    return PartSpec("rotary", {"rotary_dim": dims if dims is not None else rot["dims"], "theta": rot["base"], "pairing": "half",
                               "scaling": scaling})


def _mixer_spec(kind: str, m: dict, width: int, eps: float, prefix: str) -> PartSpec:
    if kind == "attention":
        mask = m.get("mask") or {}
        return PartSpec("rotary_sink_attention", {
            "hidden": width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "scale": m["scale"],
            "bias": False, "head_norm_eps": eps, "gate": "element", "sink": True, "window": mask.get("size"),
            "keep_first": mask.get("keep_first") or 0, "position": _rotary(m.get("rot"))}, prefix)
    if kind == "parallel":
        left, right = m["left"], m["right"]
        return PartSpec("parallel", {
            "hidden": width, "left_scale": m["left_scale"], "right_scale": m["right_scale"],
            "left": PartSpec("rotary_sink_attention", {
                "hidden": width, "heads": left["heads"], "kv_heads": left["kv_heads"], "dim": left["dim"], "vdim": left["vdim"],
                "scale": left["scale"], "bias": True, "out_bias": False, "conv": left["conv"], "gate": "head", "sink": True,
                "window": left["mask"]["size"], "position": PartSpec("none")}, prefix + "left."),
            "right": PartSpec("gated_linear_attention", {
                "hidden": width, "heads": right["heads"], "dim": right["dim"], "vdim": right["vdim"], "tau": right["tau"], "eps": eps,
                "rank": right.get("rank")}, prefix + "right.")}, prefix)
    rot = m["rot"]
    sc = rot.get("scaling")
    return PartSpec("latent_attention", {
        "hidden": width, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"], "kv_rank": m["kv_rank"],
        "q_rank": m["q_rank"], "scale": m["scale"], "rot_base": rot["base"], "rot_dims": rot.get("dims", m["rot_dim"]), "pairing": "half", "eps": eps,
        "rot_scaling": None if not sc else {"factor": sc["factor"], "low_freq_factor": sc["low"], "high_freq_factor": sc["high"],
                                            "original_max_position_embeddings": sc["original"]}}, prefix)


def _feed_forward_spec(f: dict, width: int, prefix: str) -> PartSpec:
    if f["kind"] == "dense":
        return PartSpec("gated_dense", {"hidden": width, "intermediate": f["ff"], "activation": "gelu_tanh",
                                        "names": {"gate": "gate", "up": "up", "down": "down"}}, prefix)
    r = f["router"]
    return PartSpec("routed_experts", {
        "hidden": width, "experts": r["experts"], "top": r["top"], "ff": f["expert"]["ff"], "score": "softmax", "renormalise": False,
        "scale_input": False, "activation": "swiglu", "weight_scale": float(r["scale"]) if r.get("scale") is not None else 1.0,
        "shared": {"ff": f["shared"]["ff"], "gated": True} if f.get("shared") is not None else None}, prefix)


def gebilorn_spec(cfg: GebilornConfig) -> ModelSpec:
    width, eps = cfg.width, cfg.eps
    norm = lambda name, prefix: PartSpec("rms", {"size": width, "eps": eps, "weight_name": name, "offset": 1.0}, prefix)
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"norm": norm("norm1", p), "mixer": _mixer_spec(layer["type"], layer["mixer"], width, eps, p + "mix.")}
        if layer["mlp"] is not None:
            parts["feed_forward"] = _feed_forward_spec(layer["mlp"], width, p + "mlp.")
        layers.append(LayerSpec(PartSpec("parallel_residual"), parts))
        schedule.append(ScheduleEntry(i))
    if cfg.bigram is not None:
        embedding = PartSpec("pair_table", {"vocab": cfg.vocab, "hidden": width, "name": "embed", "scale": cfg.embedding_scale,
                                            "pairs": {"name": "bigram", "buckets": cfg.bigram[0], "mul_prev": cfg.bigram[1],
                                                      "mul_cur": cfg.bigram[2]}})
    else:
        embedding = PartSpec("table", {"vocab": cfg.vocab, "hidden": width, "name": "embed", "scale": cfg.embedding_scale})
    spec = ModelSpec(
        architecture=GebilornConfig.architecture, hidden_size=width, vocab_size=cfg.vocab, embedding=embedding, layers=layers,
        schedule=schedule, final_norm=norm("final.norm", ""),
        head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": width, "name": "head", "tied_to": "embed", "softcap": cfg.logit_softcap}),
        max_position=cfg.max_position)
    spec.validate()
    return spec


register_architecture(GebilornConfig.architecture, GebilornConfig, gebilorn_spec)
