"""A feed-forward of routed experts: each token goes through the ``top`` best of ``experts`` small gated feed-forwards.

Router logits z = W_router h are float; scores are sigmoid(z) (or a softmax over the experts); the ``top`` largest
are chosen, lowest index first on ties; the weights are the chosen scores, divided by their sum only if asked. The
weight multiplies the expert's input (``scale_input``), which matters because the experts are not linear, or its
output. Options: ``correction``, a learned float per router output that is added to the scores for the choice only (the
weights use the scores without it); ``identity``, that many more router outputs after the experts' whose "expert" is
the token's input itself (no tensors); ``shared``, one more gated feed-forward of its own width that every token goes
through, its output multiplied by sigmoid(w_sg . h) if ``gated``; ``weight_scale``, a constant every weight is multiplied
by. Expert activations: "clamped_swish": g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(alpha g)
* (u + 1); "swiglu": silu(gate) * up. The experts' matrices are stacked at load into [E, 2 ff, hidden] (gate rows,
then up rows) and [E, hidden, ff]; tokens are grouped by expert on the device, so a step has no host round trip
(csrc/routed_experts.cu).
"""
from __future__ import annotations

import torch

from ..config.spec import PartSpec
from .base import FeedForward, TensorDecl, build_part, register_part


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    """params: hidden, experts, top, ff, score ("sigmoid" | "softmax"), renormalise, renormalise_eps (added to the sum),
    scale_input, activation, limit, alpha, correction (bool), identity (count), shared ({ff, gated} or None), weight_scale,
    names: router, correction, shared (prefix), shared_gate, and expert tensor names as patterns with {e} (defaults "router",
    "correction", "shared.", "shared.sg", "e{e}.gate", "e{e}.up", "e{e}.down")."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.experts, self.top, self.ff = int(p["hidden"]), int(p["experts"]), int(p["top"]), int(p["ff"])
        self.identity = int(p.get("identity") or 0)
        self.outputs = self.experts + self.identity          # what the router scores
        if not (1 <= self.top <= self.outputs) or self.top > 16:
            raise ValueError(f"top {self.top} of {self.outputs} experts is not possible (at most 16 per token)")
        self.score = p.get("score", "sigmoid")
        self.renormalise = bool(p.get("renormalise", False))
        self.renormalise_eps = float(p.get("renormalise_eps") or 0.0)
        self.correction = bool(p.get("correction", False))
        self.weight_scale = float(p["weight_scale"]) if p.get("weight_scale") is not None else 1.0
        shared = p.get("shared")
        self.shared_gated = bool(shared and shared.get("gated"))
        self.scale_input = bool(p.get("scale_input", True))
        self.activation = p.get("activation", "clamped_swish")
        self.limit = float(p.get("limit", 0.0))
        self.alpha = float(p.get("alpha", 1.702))
        names = dict(p.get("names", {}))
        self.router_name = self.prefix + names.get("router", "router")
        self.patterns = {k: self.prefix + names.get(k, "e{e}." + k) for k in ("gate", "up", "down")}
        self.correction_name = self.prefix + names.get("correction", "correction")
        self.shared_gate_name = self.prefix + names.get("shared_gate", "shared.sg")
        self.shared = None
        if shared:
            if self.activation != "swiglu":
                raise ValueError("routed_experts: a shared expert takes the swiglu activation")
            sp = self.prefix + names.get("shared", "shared.")
            self.shared = build_part("feed_forward", PartSpec("swiglu", {"hidden": self.hidden, "intermediate": int(shared["ff"]),
                                                                         "names": {"gate": "gate", "up": "up", "down": "down"}}, sp), runtime)
        self.plain = not (self.identity or self.correction or self.shared or self.renormalise_eps or self.weight_scale != 1.0)
        self.w_router = self.w_gate_up = self.w_down = self.choice_bias = None

    def kernel_needs(self):
        return {"libraries": ["moe"]}

    def tensor_decls(self):
        decls = [TensorDecl(self.router_name, (self.outputs, self.hidden))]
        if self.correction:
            decls.append(TensorDecl(self.correction_name, (self.outputs,), role="vector", init="small"))
        if self.shared is not None:
            decls += self.shared.tensor_decls()
            if self.shared_gated:
                decls.append(TensorDecl(self.shared_gate_name, (1, self.hidden)))
        for e in range(self.experts):
            decls += [TensorDecl(self.patterns["gate"].format(e=e), (self.ff, self.hidden)),
                      TensorDecl(self.patterns["up"].format(e=e), (self.ff, self.hidden)),
                      TensorDecl(self.patterns["down"].format(e=e), (self.hidden, self.ff))]
        return decls

    def load(self, tensors):
        # the shared expert's gate is one more row of the router's matrix: one product gives all the float logits
        rows = [tensors[self.router_name]] + ([tensors[self.shared_gate_name]] if self.shared_gated else [])
        self.w_router = torch.cat(rows, dim=0).contiguous()
        self.choice_bias = tensors[self.correction_name].float().contiguous() if self.correction else None
        if self.shared is not None:
            self.shared.load(tensors)
        self.w_gate_up = torch.stack([torch.cat([tensors[self.patterns["gate"].format(e=e)], tensors[self.patterns["up"].format(e=e)]], 0)
                                      for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([tensors[self.patterns["down"].format(e=e)] for e in range(self.experts)]).contiguous()

    def forward(self, h, ctx):
        rt = self.rt
        t = h.shape[0]
        logits = torch.empty((t, self.w_router.shape[0]), dtype=torch.float32, device=rt.device)
        rt.kernels.linear(h, self.w_router, logits)
        out = rt.empty_act((t, self.hidden))
        if self.plain:
            rt.kernels.routed_experts(h, logits, self.w_gate_up, self.w_down, self.top, out, score=self.score, renormalise=self.renormalise,
                                      scale_input=self.scale_input, activation=self.activation, limit=self.limit, alpha=self.alpha)
            return out
        shared = self.shared.forward(h, ctx) if self.shared is not None else None
        rt.kernels.routed_experts(h, logits, self.w_gate_up, self.w_down, self.top, out, score=self.score, renormalise=self.renormalise,
                                  scale_input=self.scale_input, activation=self.activation, limit=self.limit, alpha=self.alpha,
                                  outputs=self.outputs, choice_bias=self.choice_bias, renormalise_eps=self.renormalise_eps,
                                  shared=shared, shared_gated=self.shared_gated,
                                  **({"weight_scale": self.weight_scale} if self.weight_scale != 1.0 else {}))
        return out


@register_part("feed_forward", "table_experts")
class TableExperts(FeedForward):
    """Experts without a router: an integer table [vocab, top] gives every token id its ``top`` experts (the entries
    of a row differ), each weighing 1 / top on its output. An expert is down(act(up h)) without a gate; act is the
    square of relu. The experts' matrices are stacked at load into [E, ff, hidden] and [E, hidden, ff]; grouping by
    expert and the two products are those of the routed experts (csrc/routed_experts.cu).
    params: hidden, experts, top, ff, vocab, activation ("relu_squared"), names: table, up, down (patterns with {e})."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.experts, self.top, self.ff = int(p["hidden"]), int(p["experts"]), int(p["top"]), int(p["ff"])
        self.vocab = int(p["vocab"])
        if not (1 <= self.top <= self.experts) or self.top > 16:
            raise ValueError(f"top {self.top} of {self.experts} experts is not possible (at most 16 per token)")
        self.activation = p.get("activation", "relu_squared")
        if self.activation != "relu_squared":
            raise ValueError(f"table_experts: activation {self.activation!r} is not known (relu_squared)")
        names = dict(p.get("names", {}))
        self.table_name = self.prefix + names.get("table", "table")
        self.patterns = {k: self.prefix + names.get(k, "e{e}." + k) for k in ("up", "down")}
        self.table = self.w_up = self.w_down = None

    def kernel_needs(self):
        return {"libraries": ["moe"]}

    def tensor_decls(self):
        decls = [TensorDecl(self.table_name, (self.vocab, self.top), role="table", init=f"choice:{self.experts}")]
        for e in range(self.experts):
            decls += [TensorDecl(self.patterns["up"].format(e=e), (self.ff, self.hidden)),
                      TensorDecl(self.patterns["down"].format(e=e), (self.hidden, self.ff))]
        return decls

    def load(self, tensors):
        self.table = tensors[self.table_name].contiguous()
        if int(self.table.min()) < 0 or int(self.table.max()) >= self.experts:
            raise ValueError(f"{self.table_name}: an entry names an expert outside 0..{self.experts - 1}")
        self.w_up = torch.stack([tensors[self.patterns["up"].format(e=e)] for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([tensors[self.patterns["down"].format(e=e)] for e in range(self.experts)]).contiguous()

    def forward(self, h, ctx):
        out = self.rt.empty_act((h.shape[0], self.hidden))
        self.rt.kernels.table_experts(h, ctx.tokens, getattr(ctx, "last_token", None), self.table, self.w_up, self.w_down, self.top, out,
                                      activation=self.activation)
        return out
