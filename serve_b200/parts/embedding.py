"""Token embedding and output head.

Embedding: a row gather (serve/model.py:157,220), written into the float32
residual stream. Head: logits = x W^T without bias (model.py:159,227,231), in
float32. A tied head uses the embedding's table (the reference copies it at
conversion, serve/hf_utils/convert_hf_checkpoint.py:146-147).
"""
from __future__ import annotations

import torch

from .base import CacheNeed, Part, TensorDecl, register_part


@register_part("embedding", "table")
class TokenEmbedding(Part):
    """params: vocab, hidden, name, scale (every row is multiplied by it in float32; default 1)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab = int(spec.params["vocab"])
        self.hidden = int(spec.params["hidden"])
        self.name = self.prefix + spec.params.get("name", "weight")
        self.scale = float(spec.params.get("scale") or 1.0)
        self.table = None

    def tensor_decls(self):
        return [TensorDecl(self.name, (self.vocab, self.hidden))]

    def load(self, tensors):
        self.table = tensors[self.name]

    def forward(self, tokens, ctx):
        x = torch.empty((tokens.shape[0], self.hidden), dtype=torch.float32, device=self.rt.device)
        if self.scale != 1.0:
            self.rt.kernels.embedding(tokens, self.table, x, getattr(ctx, "last_token", None), scale=self.scale)
        else:
            self.rt.kernels.embedding(tokens, self.table, x, getattr(ctx, "last_token", None))
        return x


@register_part("embedding", "pair_table")
class PairTableEmbedding(TokenEmbedding):
    """The token's row times ``scale`` plus a row of a second table chosen by the token together with the one before it:
    row (previous id * mul_prev + id * mul_cur) mod buckets, and row ``buckets`` (the table's last) for a sequence's first
    token. The id before a portion's first token is per-request state: one number per slot, kept as an integer's bits
    in the float state pool. params: vocab, hidden, name, scale, pairs {name, buckets, mul_prev, mul_cur}."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        pairs = spec.params["pairs"]
        self.pairs_name = self.prefix + pairs.get("name", "pairs")
        self.buckets, self.mul_prev, self.mul_cur = int(pairs["buckets"]), int(pairs["mul_prev"]), int(pairs["mul_cur"])
        if self.buckets <= 0 or self.mul_prev < 0 or self.mul_cur < 0:
            raise ValueError("pair_table: buckets must be positive and the multipliers not negative")
        self.pairs = None

    def kernel_needs(self):
        return {"libraries": ["prep"]}

    def tensor_decls(self):
        return super().tensor_decls() + [TensorDecl(self.pairs_name, (self.buckets + 1, self.hidden))]

    def load(self, tensors):
        super().load(tensors)
        self.pairs = tensors[self.pairs_name]

    def cache_need(self):
        return CacheNeed(states=(("previous_token", (1,)),))

    def forward(self, tokens, ctx, cache=None):
        x = torch.empty((tokens.shape[0], self.hidden), dtype=torch.float32, device=self.rt.device)
        self.rt.kernels.embedding_pair(ctx, self.table, self.pairs, cache.states["previous_token"], self.buckets, self.mul_prev,
                                       self.mul_cur, x, scale=self.scale)
        return x


@register_part("head", "linear")
class OutputHead(Part):
    """params: vocab, hidden, name; tied_to: name of the embedding table, or None; softcap c (None: none): the logits
    become c * tanh(logits / c)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab = int(spec.params["vocab"])
        self.hidden = int(spec.params["hidden"])
        self.tied_to = spec.params.get("tied_to")
        self.own_name = self.prefix + spec.params.get("name", "weight")
        self.name = self.tied_to if self.tied_to else self.own_name
        self.softcap = float(spec.params["softcap"]) if spec.params.get("softcap") else 0.0
        self.weight = None

    def kernel_needs(self):
        return {"libraries": ["prep"]} if self.softcap else {}

    def tensor_decls(self):
        return [TensorDecl(self.name, (self.vocab, self.hidden))]

    def ignorable_tensors(self):
        return [self.own_name] if self.tied_to else []

    def load(self, tensors):
        self.weight = tensors[self.name]

    def forward(self, h, ctx):
        logits = torch.empty((h.shape[0], self.vocab), dtype=torch.float32, device=self.rt.device)
        self.rt.kernels.linear(h, self.weight, logits)
        if self.softcap:
            self.rt.kernels.softcap(logits, self.softcap)
        return logits
