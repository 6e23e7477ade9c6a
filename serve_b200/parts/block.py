"""Block arrangements: how norms, mixer and feed-forward sit on the residual stream.

"pre_norm" is the reference's block (serve/model.py:146-149):
x = x + mixer(norm1(x)); x = x + ffn(norm2(x)). The residual stream x is
float32; each sub-layer's output is handed on as a pending delta and added
inside the next norm kernel.
"""
from __future__ import annotations

from .base import Block, CacheNeed, DeferredNorm, DeltaPair, register_part


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    wants = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def fused_description(self, cache):
        """This arrangement with its parts' own descriptions, for kernels that run whole layers at once; None if a part
        has no description to give (such a layer runs part by part)."""
        out = {"kind": "pre_norm"}
        for name in self.wants:
            describe = getattr(getattr(self, name), "fused_description", None)
            if describe is None:
                return None
            out[name] = describe(cache) if name == "mixer" else describe()
        return out

    def forward(self, x, pending, ctx, cache):
        h = self.mixer_norm.forward(x, pending, ctx)
        a = self.mixer.forward(h, ctx, cache)
        h = self.feed_forward_norm.forward(x, a, ctx)
        f = self.feed_forward.forward(h, ctx)
        return x, f


@register_part("block", "pre_norm_filtered")
class PreNormFilteredBlock(Block):
    """The pre-norm arrangement with a filter over time between each norm and its sub-layer:
    x = x + mixer(filter1(norm1(x))); x = x + ffn(filter2(norm2(x))). Either filter, and the whole feed-forward half,
    may be left out. The filters' states belong to the layer's cache, beside the mixer's, under "mixer_filter.*" and
    "feed_forward_filter.*"."""

    wants = {"mixer_norm": "norm", "mixer_filter": "filter", "mixer": "mixer", "feed_forward_norm": "norm",
             "feed_forward_filter": "filter", "feed_forward": "feed_forward"}
    optional = ("mixer_filter", "feed_forward_norm", "feed_forward_filter", "feed_forward")

    def cache_need(self):
        needs = [("", self.mixer.cache_need())]
        for name in ("mixer_filter", "feed_forward_filter"):
            part = getattr(self, name)
            if part is not None:
                needs.append((name + ".", part.cache_need()))
        return CacheNeed.merged(needs)

    def forward(self, x, pending, ctx, cache):
        h = self.mixer_norm.forward(x, pending, ctx)
        if self.mixer_filter is not None:
            h = self.mixer_filter.forward(h, ctx, cache, prefix="mixer_filter.")
        a = self.mixer.forward(h, ctx, cache)
        if self.feed_forward is None:
            return x, a
        h = self.feed_forward_norm.forward(x, a, ctx)
        if self.feed_forward_filter is not None:
            h = self.feed_forward_filter.forward(h, ctx, cache, prefix="feed_forward_filter.")
        f = self.feed_forward.forward(h, ctx)
        return x, f


@register_part("block", "sandwich_norm")
class SandwichNormBlock(Block):
    """A norm before and a norm after each sub-layer: x = x + norm_b(mixer(norm(x))); x = x + norm_d(ffn(norm_c(x))).
    The feed-forward half may be left out. A sub-layer's output is handed on together with its own norm (``DeferredNorm``):
    the norm that reads the residual stream next applies it in the same kernel if it can, so no normalised delta is
    written and read in between."""

    wants = {"mixer_norm": "norm", "mixer": "mixer", "mixer_post_norm": "norm", "feed_forward_norm": "norm",
             "feed_forward": "feed_forward", "feed_forward_post_norm": "norm"}
    optional = ("feed_forward_norm", "feed_forward", "feed_forward_post_norm")

    def __init__(self, spec, runtime, parts=None):
        super().__init__(spec, runtime, parts)
        if (self.feed_forward is None) != (self.feed_forward_norm is None) or (self.feed_forward is None) != (self.feed_forward_post_norm is None):
            raise KeyError("sandwich_norm: a feed-forward comes with both of its norms, or none of the three is given")

    def forward(self, x, pending, ctx, cache):
        h = self.mixer_norm.forward(x, pending, ctx)
        a = DeferredNorm(self.mixer.forward(h, ctx, cache), self.mixer_post_norm)
        if self.feed_forward is None:
            return x, a
        h = self.feed_forward_norm.forward(x, a, ctx)
        return x, DeferredNorm(self.feed_forward.forward(h, ctx), self.feed_forward_post_norm)


@register_part("block", "parallel_residual")
class ParallelResidualBlock(Block):
    """One norm whose output both sub-layers read: h = norm(x); x = x + (mixer(h) + ffn(h)). The feed-forward may be left
    out. Both outputs travel as the pending delta (a ``DeltaPair``); the norm that reads the residual stream next adds each
    of them in float in its own kernel, or, if it cannot, gets their float sum."""

    wants = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}
    optional = ("feed_forward",)

    def forward(self, x, pending, ctx, cache):
        h = self.norm.forward(x, pending, ctx)
        a = self.mixer.forward(h, ctx, cache)
        if self.feed_forward is None:
            return x, a
        return x, DeltaPair(a, self.feed_forward.forward(h, ctx))
