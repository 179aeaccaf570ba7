"""Two mixers side by side: both read the same input, each output is RMS-normed over the model width with a plain
weight, and the result is `coef` times their sum (csrc/dyt.cu, `jv_norm_mean2`, 32-bit).

Each side keeps what it needs (pages of keys and values, a state row, ...): the pair's cache need is the tuple of its
sides' needs and it receives a tuple of cache views.  One product over the stacked input matrices serves both sides.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, TensorSpec
from .registry import MIXERS, build, register_mixer


class MixerPair(Part):
    def __init__(self, spec, prefix, ctx):
        self.spec, self.ctx = spec, ctx
        self.prefix = f"{prefix}.{spec.prefix}" if spec.prefix else prefix
        self.sides = (build(MIXERS, "mixer", spec.left, self.prefix, ctx), build(MIXERS, "mixer", spec.right, self.prefix, ctx))
        for side in self.sides:
            if not hasattr(side, "forward_projected"):
                raise ValueError(f"{self.prefix}: a side of a pair offers its input product (`in_weight`, `forward_projected`)")
        self.kernels = tuple(dict.fromkeys(("dyt",) + self.sides[0].kernels + self.sides[1].kernels))
        self.capturable = all(getattr(side, "capturable", True) for side in self.sides)
        self.w_in = self.out_w = None

    def tensor_specs(self):
        out = {}
        for side in self.sides:
            out.update(side.tensor_specs())
        for name in self.spec.names:
            out[f"{self.prefix}.{name}"] = TensorSpec((self.spec.hidden_size,), kind="vector", init="ones_normal")
        return out

    def bind(self, tensors):
        for side in self.sides:
            side.bind(tensors)
        ws = [tensors[f"{self.prefix}.{name}"].contiguous() for name in self.spec.names]
        self.out_w = (ws[0], ws[1].to(ws[0].dtype))
        ins = [side.in_weight() for side in self.sides]
        if ins[0].dtype != ins[1].dtype:
            ins = [w.to(torch.float32) for w in ins]
        self.w_in = torch.cat(ins, dim=0).contiguous()
        self.kernels = tuple(dict.fromkeys(("dyt",) + self.sides[0].kernels + self.sides[1].kernels))

    @property
    def in_rows(self):
        return self.sides[0].in_rows + self.sides[1].in_rows

    def in_weight(self):
        return self.w_in

    def cache_need(self):
        return tuple(side.cache_need() for side in self.sides)

    def tile_classes(self, page_size: int):
        out = []
        for side in self.sides:
            f = getattr(side, "tile_classes", None)
            if f is not None:
                out += list(f(page_size))
        return out

    def forward_projected(self, row, step, cache):
        n0 = self.sides[0].in_rows
        a = self.sides[0].forward_projected(row[:, :n0], step, cache[0])
        b = self.sides[1].forward_projected(row[:, n0:n0 + self.sides[1].in_rows], step, cache[1])
        return ops.norm_mean2(a, b, self.out_w[0], self.out_w[1], self.spec.eps, self.spec.coef)

    def forward(self, x, step, cache):
        return self.forward_projected(ops.linear(x, self.w_in, self.ctx.dtype), step, cache)


register_mixer("mixer_pair", MixerPair)
