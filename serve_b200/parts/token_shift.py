"""Token shift: every consumer reads its own blend of a token's input with the input of the token before it.

out[s, t] = x[t] + (x[t - 1] - x[t]) * mu[s], one float vector mu[s] per consumer; before the first token of a sequence
stand zeros. The input of a request's last token is kept as per-request state (float, shape (1, channels)), so a
portion continues where the one before stopped, wherever the prompt was cut. The blends are computed in float and
rounded once.
"""
from __future__ import annotations

import torch

from .base import CacheNeed, SequenceFilter, TensorDecl, register_part


@register_part("filter", "token_shift")
class TokenShift(SequenceFilter):
    """params: channels, mixes (tensor names of the blend vectors, relative to the prefix, in output order), state_name
    (default "shift")."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.channels = int(p["channels"])
        self.mix_names = [self.prefix + n for n in p["mixes"]]
        if not self.mix_names:
            raise ValueError("a token shift needs at least one blend")
        self.state_name = p.get("state_name", "shift")
        self.mu = None

    def kernel_needs(self):
        return {"libraries": ["seq"]}

    def tensor_decls(self):
        return [TensorDecl(n, (self.channels,), role="vector", init="normal") for n in self.mix_names]

    def load(self, tensors):
        self.mu = torch.stack([tensors[n].float() for n in self.mix_names]).contiguous()

    def cache_need(self):
        return CacheNeed(states=((self.state_name, (1, self.channels)),))

    def forward(self, x, ctx, cache, out=None, prefix: str = ""):
        if out is None:
            out = self.rt.empty_act((len(self.mix_names), x.shape[0], self.channels))
        self.rt.kernels.token_shift_mix(x, self.mu, cache.states[prefix + self.state_name], ctx, out)
        return out
