"""Rotary position encoding: inv_freq[j] = 1 / theta^(2j/dim) / scaling_factor, j < dim/2, in 32-bit
(jllm/model/common.py:51-55; the factor is linear scaling of positions).  `layout` names the pairs that turn together:
"halves" (element i with i + dim/2) or "interleaved" (2i with 2i + 1); a mixer's preparation kernel must know it.  The part only owns the table; the rotation itself is
applied to queries and keys inside the mixer's preparation kernel (csrc/rope_kv.cu), which
forms the angle position * inv_freq[j] and its cos and sin in 32-bit."""

from __future__ import annotations

import torch

from .base import Part
from .registry import register_position


class Rope(Part):
    def __init__(self, spec, prefix, ctx):
        if spec.dim % 2 or spec.dim < 2:
            raise ValueError(f"rotary dim must be even and positive, got {spec.dim}")
        self.dim, self.theta = int(spec.dim), float(spec.theta)
        self.layout = getattr(spec, "layout", "halves")
        self.factor = float(getattr(spec, "scaling_factor", 1.0))
        if self.layout not in ("halves", "interleaved") or not self.factor > 0:
            raise ValueError(f"rotation: layout {self.layout!r} or scaling factor {self.factor} is not built")
        self.wide = torch.float64 if getattr(spec, "exact_table", False) else torch.float32
        self.inv_freq = self.frequencies(self.dim, self.factor).to(ctx.device)

    def frequencies(self, dim: int, factor: float = 1.0) -> torch.Tensor:
        """theta^(-2j/dim) / factor for j < dim/2, as float32 on the CPU."""
        exponents = torch.arange(0, dim, 2, dtype=self.wide) / dim
        return (1.0 / (self.theta ** exponents) / factor).to(torch.float32)

    def table(self):
        return self.inv_freq


register_position("rope", Rope)
