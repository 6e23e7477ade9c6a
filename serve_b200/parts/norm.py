"""RMS normalisation and layer normalisation, each fused with the residual addition that precedes it.

Reference formula (serve/model.py:63-68): y = x32 * rsqrt(mean(x32^2) + eps),
cast to the model dtype, times weight. Here the residual stream itself is kept
in float32, the pending delta of the previous sub-layer is added in the same
kernel (model.py:147-148 do it as a separate op), and the product with the
weight is taken in float32 before the single rounding to the activation dtype.
"""
from __future__ import annotations

from .base import DeferredNorm, DeltaPair, Norm, TensorDecl, plain_delta, register_part


@register_part("norm", "rms")
class RMSNorm(Norm):
    """params: size, eps, weight_name (relative to prefix, default "weight"), offset (default 0: the stored weight is its
    distance from ``offset``, so the factor is offset + w, formed once at load in float)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.weight_name = self.prefix + spec.params.get("weight_name", "weight")
        self.offset = float(spec.params.get("offset") or 0.0)
        self.weight = None

    def tensor_decls(self):
        return [TensorDecl(self.weight_name, (self.size,), role="vector", init="small" if self.offset else "norm")]

    def load(self, tensors):
        self.weight = tensors[self.weight_name]
        if self.offset:
            self.weight = (self.weight.float() + self.offset).contiguous()

    def fused_description(self):
        """What a kernel that runs whole layers at once needs to know of this norm."""
        return dict(kind="rms", size=self.size, eps=self.eps, weight=self.weight)

    def forward(self, x, delta, ctx):
        out = self.rt.empty_act((x.shape[0], self.size))
        if isinstance(delta, DeltaPair) and delta.a.dtype == out.dtype and delta.b.dtype == out.dtype:
            self.rt.kernels.add2_rmsnorm(x, delta.a, delta.b, None, self.weight, self.eps, out)      # both join in this kernel, in float
            return out
        self.rt.kernels.add_rmsnorm(x, plain_delta(delta), self.weight, self.eps, out)
        return out

    def forward_rows(self, x, delta, rows, ctx):
        out = self.rt.empty_act((rows.shape[0], self.size))
        if isinstance(delta, DeltaPair) and delta.a.dtype == out.dtype and delta.b.dtype == out.dtype:
            self.rt.kernels.add2_rmsnorm(x, delta.a, delta.b, rows, self.weight, self.eps, out)
            return out
        self.rt.kernels.add_rmsnorm_rows(x, plain_delta(delta), rows, self.weight, self.eps, out)
        return out


@register_part("norm", "layer_norm")
class LayerNorm(RMSNorm):
    """y = (x - mean) / sqrt(var + eps) * weight, var the mean of the squared deviations, no bias; the same fusion with
    the residual addition, in float32. params: size, eps, weight_name."""

    def fused_description(self):
        return None     # the kernel that runs whole layers knows RMS norms only

    def _delta(self, delta):
        d = plain_delta(delta)
        return d.to(self.rt.act_dtype) if isinstance(delta, DeltaPair) else d        # (this kernel reads a delta of the activations' type)

    def forward(self, x, delta, ctx):
        out = self.rt.empty_act((x.shape[0], self.size))
        self.rt.kernels.add_layernorm(x, self._delta(delta), self.weight, self.eps, out)
        return out

    def forward_rows(self, x, delta, rows, ctx):
        out = self.rt.empty_act((rows.shape[0], self.size))
        self.rt.kernels.add_layernorm_rows(x, self._delta(delta), rows, self.weight, self.eps, out)
        return out


@register_part("norm", "dynamic_tanh")
class DynamicTanh(Norm):
    """y = tanh(alpha * x) * weight + bias, alpha a scalar: a norm without statistics, so every element stands alone. All in
    float32. The same fusion with the residual addition as the other norms; and because it is element-wise, the norm of
    the sub-layer before (a ``DeferredNorm`` whose norm is another dynamic tanh) is applied in the same kernel:
    x += tanh(alpha' a) w' + b'; y = tanh(alpha x) w + b. params: size, weight_name (bias and alpha are "<weight>.b" and
    "<weight>.alpha")."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.size = int(spec.params["size"])
        self.weight_name = self.prefix + spec.params.get("weight_name", "weight")
        self.params = None

    def kernel_needs(self):
        return {"libraries": ["prep"]}

    def tensor_decls(self):
        return [TensorDecl(self.weight_name, (self.size,), role="vector", init="norm"),
                TensorDecl(self.weight_name + ".b", (self.size,), role="vector", init="small"),
                TensorDecl(self.weight_name + ".alpha", (), role="vector", init="norm")]

    def load(self, tensors):
        import torch

        # weight, bias and alpha as one float vector [2 * size + 1]: one pointer for the kernel, alpha on the device
        self.params = torch.cat([tensors[self.weight_name].float().reshape(-1), tensors[self.weight_name + ".b"].float().reshape(-1),
                                 tensors[self.weight_name + ".alpha"].float().reshape(-1)]).contiguous()

    def _split(self, delta):
        """(tensor to add or None, the parameters of the dynamic tanh it goes through first or None)."""
        if isinstance(delta, DeferredNorm):
            if isinstance(delta.norm, DynamicTanh):
                return delta.a, delta.norm.params
            return delta.plain(), None
        return plain_delta(delta), None

    def forward(self, x, delta, ctx):
        out = self.rt.empty_act((x.shape[0], self.size))
        a, through = self._split(delta)
        self.rt.kernels.add_dynamic_tanh(x, a, through, None, self.params, out)
        return out

    def forward_rows(self, x, delta, rows, ctx):
        out = self.rt.empty_act((rows.shape[0], self.size))
        a, through = self._split(delta)
        self.rt.kernels.add_dynamic_tanh(x, a, through, rows, self.params, out)
        return out

    def apply(self, a):
        import torch

        out = torch.empty((a.shape[0], self.size), dtype=torch.float32, device=a.device)
        self.rt.kernels.add_dynamic_tanh(None, a, None, None, self.params, out)
        return out
