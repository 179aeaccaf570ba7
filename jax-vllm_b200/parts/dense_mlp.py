"""A feed-forward without a gate: down(act(up(x))), act = relu(z)^2 or the exact gelu (by name), no bias.

Like the attention mixers it offers its two products to an arrangement that packs them with another part's
(`in_weight`, `from_projection`, `out_weight`)."""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, TensorSpec
from .registry import register_feed_forward


class DenseMLP(Part):
    kernels = ("activation", "gemm_simt")

    def __init__(self, spec, prefix, ctx):
        if spec.activation not in ops.UNARY_ACTIVATIONS:
            raise ValueError(f"feed-forward: activation {spec.activation!r} is not built "
                             f"({', '.join(ops.UNARY_ACTIVATIONS)} are)")
        self.spec, self.ctx = spec, ctx
        self.prefix = f"{prefix}.{spec.prefix}" if spec.prefix else prefix
        self.in_rows = self.heads_out = spec.intermediate_size
        self.w_up = self.w_down = None

    def _names(self):
        return tuple(f"{self.prefix}.{n}" for n in self.spec.names)

    def tensor_specs(self):
        up, down = self._names()
        s = self.spec
        return {up: TensorSpec((s.intermediate_size, s.hidden_size)), down: TensorSpec((s.hidden_size, s.intermediate_size))}

    def bind(self, tensors):
        up, down = self._names()
        self.w_up = self.compute_weight(tensors[up], self.ctx).contiguous()
        self.w_down = self.compute_weight(tensors[down], self.ctx).contiguous()

    def in_weight(self) -> torch.Tensor:
        return self.w_up

    def out_weight(self) -> torch.Tensor:
        return self.w_down

    def from_projection(self, z, step, out=None):
        return ops.unary_act(z, self.spec.activation, out)

    def forward(self, x, step):
        dt = self.ctx.dtype
        return ops.linear(self.from_projection(ops.linear(x, self.w_up, dt), step), self.w_down, dt, parts_ok=True)


register_feed_forward("dense_mlp", DenseMLP)
