"""RMSNorm over the hidden axis: y = h * rsqrt(mean(h^2) + eps) * weight, in 32-bit
(jllm/model/common.py:44-48), fused with the residual sum before it.  With an `offset` the
file holds weight - offset, and stored + offset multiplies (formed once, in 32-bit,
when the weights are bound)."""

from __future__ import annotations

from .. import ops
from .base import Part, TensorSpec
from .registry import register_norm


class RMSNorm(Part):
    kernels = ("norm",)

    def __init__(self, spec, prefix, ctx):
        self.size, self.eps = spec.size, float(spec.eps)
        self.offset = float(getattr(spec, "offset", 0.0))
        self.name = f"{prefix}.{spec.name}" if prefix else spec.name
        self.ctx = ctx
        self.weight = None

    def tensor_specs(self):
        return {self.name: TensorSpec((self.size,), kind="vector", init="normal" if self.offset else "ones_normal")}

    def bind(self, tensors):
        w = tensors[self.name]
        self.weight = (w.float() + self.offset).contiguous() if self.offset else w.contiguous()

    def norm(self, h, delta=None, out_dtype=None):
        """x = norm(h + delta); h is updated in place with the sum.  `out_dtype`: the type of x (the compute type
        by default; float32 for a reader that goes on in 32-bit)."""
        return ops.rmsnorm(h, self.weight, self.eps, out_dtype or self.ctx.dtype, delta=delta)

    def gather(self, h, delta, rows):
        """x[i] = norm(h[rows[i]] + delta[rows[i]]); h is left as it is."""
        return ops.rmsnorm(h, self.weight, self.eps, self.ctx.dtype, delta=delta, rows=rows)


register_norm("rmsnorm", RMSNorm)


class DynamicTanh(Part):
    """y = tanh(alpha * h) * weight + bias, element by element in 32-bit: no mean, no variance.  Tensors `<name>`
    (weight), `<name>.b` (bias) and `<name>.alpha` (one number).  `eps` of the spec is not used.  The residual sum
    before it, plain or through a gate (`ops.GatedDelta`), is made in the same pass (csrc/dyt.cu)."""

    kernels = ("dyt",)

    def __init__(self, spec, prefix, ctx):
        self.size = spec.size
        self.name = f"{prefix}.{spec.name}" if prefix else spec.name
        self.ctx = ctx
        self.weight = self.bias = None
        self.alpha = 0.0

    def tensor_specs(self):
        return {self.name: TensorSpec((self.size,), kind="vector", init="ones_normal"),
                f"{self.name}.b": TensorSpec((self.size,), kind="vector", init="normal"),
                f"{self.name}.alpha": TensorSpec((), kind="vector", init="ones_normal")}

    def bind(self, tensors):
        self.weight = tensors[self.name].contiguous()
        self.bias = tensors[f"{self.name}.b"].to(self.weight.dtype).contiguous()
        self.alpha = float(tensors[f"{self.name}.alpha"].float().item())

    def norm(self, h, delta=None, out_dtype=None):
        return ops.gated_add_dyt(h, delta, self.alpha, self.weight, self.bias, out_dtype or self.ctx.dtype)

    def gather(self, h, delta, rows):
        return ops.gated_add_dyt(h, delta, self.alpha, self.weight, self.bias, self.ctx.dtype, rows=rows)


register_norm("dyt", DynamicTanh)
