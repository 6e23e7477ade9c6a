"""Typed configuration of the Lilunex decoder, read from its config.json.

The file gives ``width``, ``vocab``, ``norm.eps``, ``embedding.scale`` and ``layers``. A layer names its mixer
(``type``: "wkv", "attention" or "delta"), the mixer's sizes and constants (``mixer``) and its feed-forward (``mlp``: an
object of kind "dense" or "moe", or null for a layer without one). An attention layer's ``mixer.kv_from`` = j makes it
read the keys and values that layer j cached instead of projecting its own. Every size and constant is taken from the
file; nothing is assumed equal between layers. ``max_position`` (the longest sequence the engine plans for) is optional.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Tuple

from .bapavik import _need, _positive
from .base import ConfigError, ModelConfig

_MIXER_KEYS = {
    "wkv": ("heads", "dim"),
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
    "delta": ("heads", "kv_heads", "dim", "vdim", "conv"),
}


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
        identity = f["router"].get("identity") or 0
        if not isinstance(identity, int) or identity < 0:
            raise ConfigError(f"{where}.router.identity must be a count, got {identity!r}")
        if f["router"]["top"] > f["router"]["experts"] + identity:
            raise ConfigError(f"{where}.router: top exceeds the experts there are")
        if f.get("shared") is not None:
            _need(f["shared"], ("ff",), where + ".shared")
            _positive(f["shared"], ("ff",), where + ".shared")
    else:
        raise ConfigError(f"{where}.kind {f['kind']!r} is not known (dense, moe)")


@dataclass(frozen=True)
class LilunexConfig(ModelConfig):
    width: int
    vocab: int
    eps: float
    embedding_scale: float
    layers: Tuple[Dict[str, Any], ...]
    max_position: int = 1 << 17

    architecture = "Lilunex"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LilunexConfig":
        _need(d, ("width", "vocab", "norm", "layers"), "config.json")
        _need(d["norm"], ("eps",), "norm")
        _positive(d, ("width", "vocab"), "config.json")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for i, layer in enumerate(d["layers"]):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            kind = layer["type"]
            if kind not in _MIXER_KEYS:
                raise ConfigError(f"{where}.type {kind!r} is not known ({', '.join(sorted(_MIXER_KEYS))})")
            m = layer["mixer"]
            _need(m, _MIXER_KEYS[kind], where + ".mixer")
            if kind == "wkv":
                _positive(m, ("heads", "dim"), where + ".mixer")
            elif kind == "delta":
                _positive(m, ("heads", "kv_heads", "dim", "vdim", "conv"), where + ".mixer")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{where}.mixer: heads must be a multiple of kv_heads")
            else:
                _positive(m, ("heads", "kv_heads", "dim", "vdim"), where + ".mixer")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{where}.mixer: heads must be a multiple of kv_heads")
                if m.get("mask") is not None:       # without a mask every earlier position is seen
                    _need(m["mask"], ("size",), where + ".mixer.mask")
                    _positive(m["mask"], ("size",), where + ".mixer.mask")
                    keep = m["mask"].get("keep_first") or 0
                    if not isinstance(keep, int) or keep < 0:
                        raise ConfigError(f"{where}.mixer.mask.keep_first must be a count, got {keep!r}")
                if m.get("rot") is not None:        # without a rotation queries and keys carry no position
                    _need(m["rot"], ("base", "dims"), where + ".mixer.rot")
                    if not isinstance(m["rot"]["dims"], int) or m["rot"]["dims"] < 0 or m["rot"]["dims"] % 2 or m["rot"]["dims"] > m["dim"]:
                        raise ConfigError(f"{where}.mixer.rot.dims must be even and at most dim")
                    if m["rot"].get("scaling") is not None:
                        _need(m["rot"]["scaling"], ("factor",), where + ".mixer.rot.scaling")
                        if not float(m["rot"]["scaling"]["factor"]) > 0:
                            raise ConfigError(f"{where}.mixer.rot.scaling.factor must be positive")
                src = m.get("kv_from")
                if src is not None:
                    if not isinstance(src, int) or not (0 <= src < i):
                        raise ConfigError(f"{where}.mixer.kv_from must name an earlier layer, got {src!r}")
                    other = layers[src]
                    if other["type"] != "attention" or other["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{where}.mixer.kv_from names layer {src}, which caches no keys of its own")
                    for key in ("kv_heads", "dim", "vdim"):
                        if other["mixer"][key] != m[key]:
                            raise ConfigError(f"{where}.mixer.{key} differs from that of layer {src}, whose keys and values it reads")
            f = layer.get("mlp")
            if f is not None:
                _check_mlp(f, where + ".mlp")
            layers.append(copy.deepcopy({"type": kind, "mixer": m, "mlp": f}))
        eps = float(d["norm"]["eps"])
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        scale = 1.0
        if d.get("embedding") is not None:
            _need(d["embedding"], ("scale",), "embedding")
            scale = float(d["embedding"]["scale"])
        return cls(width=int(d["width"]), vocab=int(d["vocab"]), eps=eps, embedding_scale=scale, layers=tuple(layers),
                   max_position=int(d.get("max_position") or (1 << 17)))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.eps},
                "embedding": {"scale": self.embedding_scale}, "layers": copy.deepcopy(list(self.layers)),
                "max_position": self.max_position}
