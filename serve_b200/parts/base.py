"""Interfaces and registries of the parts a layer is put together from.

Five kinds of part exist: mixer (attention here), feed-forward, norm, position
encoding and block arrangement, plus the embedding and the output head that
bracket the layers. Each kind has a registry from a name to a class; a
``PartSpec`` (kind + params + tensor-name prefix) picks and parametrises one.
A part never looks at a model configuration: everything it needs is in its
params, and everything it runs goes through the kernels object it is given.

Adding a part means writing a class with the interface below and registering it
under a new name; the framework's files do not change.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple

from ..config.spec import PartSpec


@dataclass(frozen=True)
class TensorDecl:
    """A tensor a part wants from the weight file.

    role: "matrix" is cast to the compute dtype (bfloat16 or float32);
          "vector" keeps 32-bit storage if the file has it, else the compute dtype;
          "table" is an integer table, kept as int32.
    init: how the random-weights mode fills it ("normal" or "norm").
    """

    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"


@dataclass(frozen=True)
class CacheNeed:
    """What one execution of a mixer wants from the cache manager.

    A mixer with keys and values in pages gives kv_heads/head_dim, a window if
    only the last ``window`` keys are ever read, and ``chunk`` if a query only
    reads the keys of its own block of ``chunk`` positions (counted from the
    start of the sequence). A mixer with per-request state of fixed size gives
    ``state_shape`` (elements of float32 per request); a layer with several
    such states (a recurrence and the tails of its convolutions, say) names
    them in ``states``, a tuple of (name, shape) pairs. Any may be absent.
    ``shared_kv``: the mixer's values are (a part of) its cached key rows, so the
    cache keeps one tensor per execution and hands it out as both.
    """

    kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Optional[Tuple[int, ...]] = None
    chunk: Optional[int] = None
    states: Tuple[Tuple[str, Tuple[int, ...]], ...] = ()
    shared_kv: bool = False      # keys and values are the same cached rows: one tensor serves as both
    keep_first: int = 0          # with a window: the sequence's first ``keep_first`` keys stay readable for good

    @property
    def has_pages(self) -> bool:
        return self.kv_heads > 0 and self.head_dim > 0

    def group_key(self) -> Tuple:
        """Executions with equal keys share page geometry, a pool and block tables."""
        return ((self.kv_heads, self.head_dim, self.window, self.chunk) + (("shared_kv",) if self.shared_kv else ())
                + (("keep_first", self.keep_first) if self.keep_first else ()))

    def covering(self, reader: "Optional[CacheNeed]") -> "CacheNeed":
        """This need, widened so that ``reader`` (the need of another execution that reads the same pages with a mask of
        its own) finds every key it may look at: the longer window (none, if either has none), the larger count of kept
        first keys, and a block of positions only if both read the same one."""
        if reader is None or not reader.has_pages:
            return self
        if (reader.kv_heads, reader.head_dim, reader.shared_kv) != (self.kv_heads, self.head_dim, self.shared_kv):
            raise ValueError("an execution that reads another's pages must have its page geometry")
        window = None if self.window is None or reader.window is None else max(self.window, reader.window)
        chunk = self.chunk if self.chunk == reader.chunk else None
        keep = max(self.keep_first, reader.keep_first) if window is not None else 0
        return CacheNeed(self.kv_heads, self.head_dim, window, self.state_shape, chunk, self.states, self.shared_kv, keep)

    @staticmethod
    def merged(needs: "List[Tuple[str, Optional[CacheNeed]]]") -> "Optional[CacheNeed]":
        """One need out of those of several parts of a layer, each with the prefix its state names get. At most
        one of them may want pages."""
        paged = [n for _, n in needs if n is not None and n.has_pages]
        if len(paged) > 1:
            raise ValueError("a layer can own the pages of one mixer only")
        states = []
        for prefix, n in needs:
            if n is None:
                continue
            if n.state_shape is not None:
                states.append((prefix + "state", tuple(n.state_shape)))
            states.extend((prefix + name, tuple(shape)) for name, shape in n.states)
        if not paged and not states:
            return None
        p = paged[0] if paged else CacheNeed()
        return CacheNeed(p.kv_heads, p.head_dim, p.window, None, p.chunk, tuple(states), p.shared_kv, p.keep_first)


class Part:
    """Base of all parts. ``spec.params`` holds every size and constant."""

    def __init__(self, spec: PartSpec, runtime):
        self.spec = spec
        self.prefix = spec.prefix
        self.rt = runtime  # serve_b200.engine.runtime.Runtime: kernels, device, dtypes

    def tensor_decls(self) -> List[TensorDecl]:
        return []

    def ignorable_tensors(self) -> List[str]:
        """Names that may be in the file without being used (no 'unexpected' error)."""
        return []

    def load(self, tensors: Dict[str, Any]) -> None:
        """Take the declared tensors (already on the device, in their kept dtype)."""

    def kernel_needs(self) -> Dict[str, Any]:
        """Which compiled libraries this part will call: {"attention_head_dims": [...], "libraries": [names]}. The engine
        builds what all parts of a model name side by side before the first step; a part that names nothing has its
        libraries built when it first calls them."""
        return {}


class Mixer(Part):
    def cache_need(self) -> Optional[CacheNeed]:
        return None

    # A mixer whose last step is a plain output projection may offer it apart: ``mix_into`` writes what the projection
    # reads (times ``scale``) into ``out``, a [T, mixed_size] column slice, and ``output_weight`` is the projection's
    # [hidden, mixed_size] matrix. An arrangement of several such mixers then projects all of them with one product.
    mixed_size: Optional[int] = None

    def mix_into(self, h, ctx, cache, out, scale: float = 1.0) -> None:
        raise NotImplementedError

    def output_weight(self):
        raise NotImplementedError

    def forward(self, h, ctx, cache):
        """h: [T, hidden] activations -> [T, hidden] activations (the residual delta).

        ``ctx`` is the step's StepContext; ``cache`` the CacheView of this
        execution (None if the mixer declared no need). ``cache.writes`` tells
        whether this execution owns the cache or only reads another's.
        """
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h, ctx):
        raise NotImplementedError


class DeferredNorm:
    """A sub-layer's output ``a`` that still has to go through a norm of its own before it joins the residual stream
    (an arrangement with norms after its sub-layers hands these on as the pending delta). A norm that can apply
    ``norm`` inside its own kernel takes the pair as it is; any other asks for ``plain()``, the normalised delta as a
    float32 tensor."""

    def __init__(self, a, norm):
        self.a, self.norm = a, norm

    def plain(self):
        return self.norm.apply(self.a)


class DeltaPair:
    """The outputs of two sub-layers that read the same norm and both still have to join the residual stream. A norm that
    can add both in its own kernel takes the pair as it is; any other asks for ``plain()``, their float sum."""

    def __init__(self, a, b):
        self.a, self.b = a, b

    def plain(self):
        return self.a.float() + self.b.float()


def plain_delta(delta):
    """A pending delta as a tensor (or None), whatever form it was handed on in."""
    return delta.plain() if isinstance(delta, (DeferredNorm, DeltaPair)) else delta


class Norm(Part):
    def forward(self, x, delta, ctx):
        """x (float32 residual, updated in place with ``delta`` if given) -> normalised activations."""
        raise NotImplementedError

    def forward_rows(self, x, delta, rows, ctx):
        """As forward, but only for the rows listed (no update of x)."""
        raise NotImplementedError

    def apply(self, a):
        """The norm of activations that are not the residual stream (a sub-layer's output): [T, size] -> float32 [T, size]."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Held by a mixer; describes how positions enter queries and keys."""


class SequenceFilter(Part):
    """A filter over time on the input of a sub-layer or inside a mixer (a short convolution): it may keep a state."""

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def forward(self, x, ctx, cache, out=None, prefix: str = ""):
        """x [T, C] -> [T, C]; ``cache.states[prefix + name]`` holds this filter's state."""
        raise NotImplementedError


class Block(Part):
    """An arrangement of parts around the residual stream.

    ``wants`` maps the names the arrangement gives its parts to their families
    ("mixer", "feed_forward", "norm", ...); the layer description brings one
    PartSpec per name, the constructor builds each and keeps it as an attribute of
    that name. ``spec.params`` holds the arrangement's own constants, if it has
    any. The part named "mixer", if there is one, is the one whose cache the
    layer owns; an arrangement whose cached part has another name overrides
    ``cache_need``.
    """

    wants: Dict[str, str] = {}
    optional: Tuple[str, ...] = ()      # names of ``wants`` that a layer may leave out (the attribute is then None)

    def __init__(self, spec: PartSpec, runtime, parts: Optional[Dict[str, PartSpec]] = None):
        super().__init__(spec, runtime)
        given = dict(parts or {})
        missing = [n for n in self.wants if n not in given and n not in self.optional]
        extra = [n for n in given if n not in self.wants]
        if missing or extra:
            raise KeyError(f"block {spec.kind!r} arranges the parts {sorted(self.wants)}; the layer description "
                           f"lacks {sorted(missing)} and has {sorted(extra)} beyond them")
        self._built = []
        for name, family in self.wants.items():
            if name not in given:
                setattr(self, name, None)
                continue
            part = build_part(family, given[name], runtime)
            setattr(self, name, part)
            self._built.append(part)

    def parts(self) -> List[Part]:
        return list(self._built)

    def cache_need(self) -> Optional[CacheNeed]:
        mixer = getattr(self, "mixer", None)
        return mixer.cache_need() if mixer is not None else None

    def forward(self, x, pending, ctx, cache):
        """(x, pending) -> (x, pending); ``pending`` is a delta not yet added to x."""
        raise NotImplementedError


_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "mixer": {},
    "feed_forward": {},
    "norm": {},
    "position": {},
    "filter": {},
    "block": {},
    "embedding": {},
    "head": {},
}


def register_part(family: str, name: str):
    """Class decorator: make a part constructible from ``PartSpec(kind=name)``."""
    if family not in _REGISTRIES:
        raise KeyError(f"unknown part family {family!r}; families: {', '.join(_REGISTRIES)}")

    def deco(cls):
        _REGISTRIES[family][name] = cls
        return cls

    return deco


def build_part(family: str, spec: PartSpec, runtime, **extra):
    try:
        cls = _REGISTRIES[family][spec.kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES.get(family, {}))) or "(none)"
        raise KeyError(f"no {family} part named {spec.kind!r}; registered: {known}") from None
    return cls(spec, runtime, **extra)


def registered(family: str) -> Tuple[str, ...]:
    return tuple(sorted(_REGISTRIES[family]))
