"""Dense feed-forwards: gated, down( act(gate x, up x) ) with act = silu(g) * u (SwiGLU) or a clamped form, and plain,
down( act(up x) ).

Reference: serve/model.py:80-85 (w1 = gate, w3 = up, w2 = down, no biases).
Gate and up weights are fused at load into one [2*I, hidden] matrix so that one
matrix product feeds the activation kernel.
"""
from __future__ import annotations

import torch

from .base import FeedForward, TensorDecl, register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """params: hidden, intermediate, names (gate/up/down tensor names relative to prefix)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden"])
        self.intermediate = int(p["intermediate"])
        names = p.get("names", {})
        self.gate_name = self.prefix + names.get("gate", "gate_proj.weight")
        self.up_name = self.prefix + names.get("up", "up_proj.weight")
        self.down_name = self.prefix + names.get("down", "down_proj.weight")
        self.w_gate_up = None
        self.w_down = None

    def tensor_decls(self):
        return [
            TensorDecl(self.gate_name, (self.intermediate, self.hidden)),
            TensorDecl(self.up_name, (self.intermediate, self.hidden)),
            TensorDecl(self.down_name, (self.hidden, self.intermediate)),
        ]

    def load(self, tensors):
        self.w_gate_up = torch.cat([tensors[self.gate_name], tensors[self.up_name]], dim=0).contiguous()
        self.w_down = tensors[self.down_name].contiguous()

    def fused_description(self):
        """What a kernel that runs whole layers at once needs to know of this feed-forward."""
        return dict(kind="swiglu", hidden=self.hidden, intermediate=self.intermediate, w_gate_up=self.w_gate_up, w_down=self.w_down)

    def forward(self, h, ctx):
        rt = self.rt
        t = h.shape[0]
        act = rt.empty_act((t, self.intermediate))
        rt.kernels.gate_up_swiglu(h, self.w_gate_up, act)
        out = rt.empty_act((t, self.hidden))
        rt.kernels.linear(act, self.w_down, out)
        return out


@register_part("feed_forward", "gated_dense")
class GatedDense(SwiGLU):
    """The same three matrices with the activation as a parameter. params: hidden, intermediate, names, activation
    ("swiglu" | "clamped_swish" | "gelu_tanh"), limit, alpha. clamped_swish: g <- min(g, limit), u <- clamp(u, -limit, limit),
    g * sigmoid(alpha g) * (u + 1), computed in float32 on the float sums of the product where that is fused. gelu_tanh:
    0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3))) * u."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.activation = p.get("activation", "swiglu")
        if self.activation not in ("swiglu", "clamped_swish", "gelu_tanh"):
            raise ValueError(f"gated_dense: activation {self.activation!r} is not known (swiglu, clamped_swish, gelu_tanh)")
        self.limit = float(p.get("limit") or 0.0)
        self.alpha = float(p.get("alpha") or 1.0)

    def fused_description(self):
        return None if self.activation != "swiglu" else super().fused_description()

    def kernel_needs(self):
        return {"libraries": ["prep"]} if self.activation != "swiglu" else {}

    def forward(self, h, ctx):
        if self.activation == "swiglu":
            return super().forward(h, ctx)
        rt = self.rt
        t = h.shape[0]
        act = rt.empty_act((t, self.intermediate))
        rt.kernels.gate_up_activation(h, self.w_gate_up, act, self.activation, self.limit, self.alpha)
        out = rt.empty_act((t, self.hidden))
        rt.kernels.linear(act, self.w_down, out)
        return out


@register_part("feed_forward", "plain_dense")
class PlainDense(FeedForward):
    """down(act(up h)) without a gate. params: hidden, intermediate, activation ("relu_squared" | "gelu_tanh" | "silu" | "tanh"),
    names (up/down tensor names relative to prefix). The activation is computed in float32 and rounded once."""

    ACTIVATIONS = ("relu_squared", "gelu_tanh", "silu", "tanh")

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.intermediate = int(p["hidden"]), int(p["intermediate"])
        self.activation = p.get("activation", "relu_squared")
        if self.activation not in self.ACTIVATIONS:
            raise ValueError(f"plain_dense: activation {self.activation!r} is not known ({', '.join(self.ACTIVATIONS)})")
        names = p.get("names", {})
        self.up_name, self.down_name = self.prefix + names.get("up", "up"), self.prefix + names.get("down", "down")
        self.w_up = self.w_down = None

    def kernel_needs(self):
        return {"libraries": ["prep"]}

    def tensor_decls(self):
        return [TensorDecl(self.up_name, (self.intermediate, self.hidden)), TensorDecl(self.down_name, (self.hidden, self.intermediate))]

    def load(self, tensors):
        self.w_up, self.w_down = tensors[self.up_name].contiguous(), tensors[self.down_name].contiguous()

    def forward(self, h, ctx):
        rt = self.rt
        act = rt.empty_act((h.shape[0], self.intermediate))
        rt.kernels.linear_activation(h, self.w_up, act, self.activation)
        out = rt.empty_act((h.shape[0], self.hidden))
        rt.kernels.linear(act, self.w_down, out)
        return out
