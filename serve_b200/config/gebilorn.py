"""Typed configuration of the Gebilorn decoder, read from its config.json.

The file gives ``width``, ``vocab``, ``norm.eps``, ``embedding`` (``scale``, and ``bigram`` with ``buckets``, ``mul_prev``,
``mul_cur`` for the table of token pairs), ``logit_softcap`` and ``layers``. A layer names its mixer (``type``: "attention",
"parallel" or "latent_attention"), the mixer's sizes and constants (``mixer``) and its feed-forward (``mlp``: an object of
kind "dense" or "moe", or null for a layer without one). Every size and constant is taken from the file; nothing is
assumed equal between layers. What a file may leave out: ``embedding.bigram`` (no pair table), ``logit_softcap`` (no cap),
an attention's ``mask`` (every earlier position is seen), ``mask.keep_first`` (none kept), ``rot`` (no rotation),
``rot.scaling`` (frequencies as they are), a router's ``scale`` (1), an expert layer's ``shared``. ``max_position`` (the
longest sequence the engine plans for) is optional.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .bapavik import _need, _positive
from .base import ConfigError, ModelConfig


def _number(d, keys, where: str, positive: bool = True) -> None:
    for k in keys:
        if isinstance(d[k], bool) or not isinstance(d[k], (int, float)) or (positive and not d[k] > 0):
            raise ConfigError(f"{where}.{k} must be a {'positive ' if positive else ''}number, got {d[k]!r}")


def _check_rot(rot, limit: int, where: str, dims_optional: bool = False) -> None:
    _need(rot, ("base",) if dims_optional else ("base", "dims"), where)
    _number(rot, ("base",), where)
    dims = rot.get("dims", limit)
    if not isinstance(dims, int) or isinstance(dims, bool) or dims < 0 or dims % 2 or dims > limit:
        raise ConfigError(f"{where}.dims must be even and at most {limit}")
    if rot.get("scaling") is not None:
        _need(rot["scaling"], ("factor", "low", "high", "original"), where + ".scaling")
        _number(rot["scaling"], ("factor", "low", "high", "original"), where + ".scaling")
        if rot["scaling"]["high"] == rot["scaling"]["low"]:
            raise ConfigError(f"{where}.scaling: low and high must differ")


def _check_heads(m, where: str) -> None:
    _need(m, ("heads", "kv_heads", "dim", "vdim", "scale"), where)
    _positive(m, ("heads", "kv_heads", "dim", "vdim"), where)
    _number(m, ("scale",), where)
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{where}: heads must be a multiple of kv_heads")


def _check_mask(mask, where: str, keep_allowed: bool) -> None:
    _need(mask, ("size",), where)
    _positive(mask, ("size",), where)
    keep = mask.get("keep_first") or 0
    if not isinstance(keep, int) or keep < 0 or (keep and not keep_allowed):
        raise ConfigError(f"{where}.keep_first must be a count{'' if keep_allowed else ' (this mixer keeps none)'}, got {keep!r}")


def _check_mixer(kind: str, m, where: str) -> None:
    if kind == "attention":
        _check_heads(m, where)
        if m.get("mask") is not None:
            _check_mask(m["mask"], where + ".mask", True)
        if m.get("rot") is not None:
            _check_rot(m["rot"], m["dim"], where + ".rot")
    elif kind == "parallel":
        _need(m, ("left", "right", "left_scale", "right_scale"), where)
        _number(m, ("left_scale", "right_scale"), where, positive=False)
        left, right = m["left"], m["right"]
        _check_heads(left, where + ".left")
        _need(left, ("conv", "mask"), where + ".left")
        _positive(left, ("conv",), where + ".left")
        if left["conv"] > 16:
            raise ConfigError(f"{where}.left.conv: at most 16 taps")
        _check_mask(left["mask"], where + ".left.mask", False)
        _need(right, ("heads", "dim", "vdim", "tau"), where + ".right")
        _positive(right, ("heads", "dim", "vdim"), where + ".right")
        _number(right, ("tau",), where + ".right")
    elif kind == "latent_attention":
        _need(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot"), where)
        _positive(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"), where)
        _number(m, ("scale",), where)
        if m["rot_dim"] % 2:
            raise ConfigError(f"{where}.rot_dim must be even")
        _check_rot(m["rot"], m["rot_dim"], where + ".rot", dims_optional=True)      # (rot.dims, if the file names it, may be less than rot_dim)
    else:
        raise ConfigError(f"{where}: type {kind!r} is not known (attention, parallel, latent_attention)")


def _check_mlp(f, where: str) -> None:
    _need(f, ("kind",), where)
    if f["kind"] == "dense":
        _need(f, ("ff",), where)
        _positive(f, ("ff",), where)
    elif f["kind"] == "moe":
        _need(f, ("expert", "router"), where)
        _need(f["expert"], ("ff",), where + ".expert")
        _need(f["router"], ("experts", "top"), where + ".router")
        _positive(f["expert"], ("ff",), where + ".expert")
        _positive(f["router"], ("experts", "top"), where + ".router")
        if f["router"]["top"] > f["router"]["experts"]:
            raise ConfigError(f"{where}.router: top exceeds the experts there are")
        if f["router"].get("scale") is not None:
            _number(f["router"], ("scale",), where + ".router")
        if f.get("shared") is not None:
            _need(f["shared"], ("ff",), where + ".shared")
            _positive(f["shared"], ("ff",), where + ".shared")
    else:
        raise ConfigError(f"{where}.kind {f['kind']!r} is not known (dense, moe)")


@dataclass(frozen=True)
class GebilornConfig(ModelConfig):
    width: int
    vocab: int
    eps: float
    embedding_scale: float
    bigram: Optional[Tuple[int, int, int]]        # (buckets, mul_prev, mul_cur) or None
    logit_softcap: Optional[float]
    layers: Tuple[Dict[str, Any], ...]
    max_position: int = 1 << 17

    architecture = "Gebilorn"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GebilornConfig":
        _need(d, ("width", "vocab", "norm", "layers"), "config.json")
        _need(d["norm"], ("eps",), "norm")
        _positive(d, ("width", "vocab"), "config.json")
        _number(d["norm"], ("eps",), "norm")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for i, layer in enumerate(d["layers"]):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            _check_mixer(layer["type"], layer["mixer"], where + ".mixer")
            f = layer.get("mlp")
            if f is not None:
                _check_mlp(f, where + ".mlp")
            layers.append(copy.deepcopy({"type": layer["type"], "mixer": layer["mixer"], "mlp": f}))
        emb = d.get("embedding") or {}
        scale = 1.0
        if emb.get("scale") is not None:
            _number(emb, ("scale",), "embedding", positive=False)
            scale = float(emb["scale"])
        bigram = None
        if emb.get("bigram") is not None:
            b = emb["bigram"]
            _need(b, ("buckets", "mul_prev", "mul_cur"), "embedding.bigram")
            _positive(b, ("buckets",), "embedding.bigram")
            for k in ("mul_prev", "mul_cur"):
                if not isinstance(b[k], int) or isinstance(b[k], bool) or b[k] < 0:
                    raise ConfigError(f"embedding.bigram.{k} must be a count, got {b[k]!r}")
            bigram = (b["buckets"], b["mul_prev"], b["mul_cur"])
        cap = d.get("logit_softcap")
        if cap is not None:
            _number(d, ("logit_softcap",), "config.json")
        return cls(width=int(d["width"]), vocab=int(d["vocab"]), eps=float(d["norm"]["eps"]), embedding_scale=scale, bigram=bigram,
                   logit_softcap=float(cap) if cap is not None else None, layers=tuple(layers),
                   max_position=int(d.get("max_position") or (1 << 17)))

    def to_dict(self) -> Dict[str, Any]:
        emb: Dict[str, Any] = {"scale": self.embedding_scale}
        if self.bigram is not None:
            emb["bigram"] = {"buckets": self.bigram[0], "mul_prev": self.bigram[1], "mul_cur": self.bigram[2]}
        out = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.eps},
               "embedding": emb, "layers": copy.deepcopy(list(self.layers)), "max_position": self.max_position}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        return out
