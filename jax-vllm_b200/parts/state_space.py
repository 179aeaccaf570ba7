"""A Mamba-2 mixer (state-space duality): a matrix state per head, carried from token to token.

    row  = x @ W_in^T                          laid out [z: inner | x: inner | B: G*N | C: G*N | dt: heads], inner = H * E
    xBC  = silu(conv(x | B | C) + bias)        a short causal convolution per channel     csrc/short_conv.cu
    dt   = softplus(dt + dt_bias);  a = exp(-exp(A_log) * dt)                             csrc/mamba2.cu, 32-bit
    S   <- a S + dt B x^T,  y = S^T C + D x    per head, S [N, E]; head h reads B, C of group h // (H / G)
                                               csrc/recurrent.cu: the scan of a matrix state with key dt * B, query C
                                               and the decay a in every key channel
    out  = (norm_groups x RMSNorm)(y * silu(z)) * weight @ W_o^T        the gate comes before the norm

State per request (`FixedStateNeed`, in a state slot, zeroed at admission): the last taps - 1 inputs of the
convolution and the matrices S, both 32-bit.  A portion of a prompt starts from what the portion before left; a
decoded token is a portion of one.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import FixedStateNeed, Part, TensorSpec
from .registry import register_mixer


class StateSpace(Part):
    kernels = ("short_conv", "mamba2", "recurrent", "gemm_simt")

    def __init__(self, spec, prefix, ctx):
        self.spec, self.ctx = spec, ctx
        self.prefix = f"{prefix}.{spec.prefix}" if spec.prefix else prefix
        self.h, self.e, self.n = int(spec.num_heads), int(spec.value_dim), int(spec.state_dim)
        self.g, self.ng, self.taps = int(spec.groups), int(spec.norm_groups), int(spec.conv_taps)
        self.inner = self.h * self.e
        if min(self.h, self.e, self.n, self.g, self.ng) < 1 or self.h % self.g or self.inner % self.ng:
            raise ValueError(f"state-space mixer: {self.h} heads of {self.e} do not fit {self.g} groups and "
                             f"{self.ng} norm groups")
        if self.n > ops.SCAN_MAX_KEY:
            raise ValueError(f"state-space mixer: a state of {self.n} channels is not built (up to {ops.SCAN_MAX_KEY})")
        if not 1 <= self.taps <= ops.SHORT_CONV_MAX_TAPS:
            raise ValueError(f"state-space mixer: a convolution of {self.taps} taps is not built")
        keys = ("in", "conv", "conv_b", "dt_bias", "a_log", "skip", "norm", "o")
        self.names = {k: f"{self.prefix}.{n}" for k, n in zip(keys, spec.names)}
        self.conv_channels = self.inner + 2 * self.g * self.n
        self.in_rows = 2 * self.inner + 2 * self.g * self.n + self.h
        self.heads_out = self.inner
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.skip = self.norm = None

    def tensor_specs(self):
        n, W = self.names, self.spec.hidden_size
        vec = lambda size, init="normal": TensorSpec((size,), kind="vector", init=init)
        return {n["in"]: TensorSpec((self.in_rows, W)), n["conv"]: TensorSpec((self.conv_channels, self.taps), kind="vector"),
                n["conv_b"]: vec(self.conv_channels), n["dt_bias"]: vec(self.h), n["a_log"]: vec(self.h), n["skip"]: vec(self.h),
                n["norm"]: vec(self.inner, "ones_normal"), n["o"]: TensorSpec((W, self.inner))}

    def bind(self, tensors):
        n = self.names
        self.w_in = self.compute_weight(tensors[n["in"]], self.ctx).contiguous()
        self.w_o = self.compute_weight(tensors[n["o"]], self.ctx).contiguous()
        self.conv_w = tensors[n["conv"]].contiguous()
        self.conv_b = tensors[n["conv_b"]].to(self.conv_w.dtype).contiguous()
        self.dt_bias = tensors[n["dt_bias"]].contiguous()
        self.a_log = tensors[n["a_log"]].to(self.dt_bias.dtype).contiguous()
        self.skip = tensors[n["skip"]].contiguous()
        self.norm = tensors[n["norm"]].to(self.skip.dtype).contiguous()

    def cache_need(self):
        # one row per request: the matrices of all heads, then the convolution's last taps - 1 inputs
        return FixedStateNeed((self.h * self.n * self.e + (self.taps - 1) * self.conv_channels,), torch.float32)

    def in_weight(self) -> torch.Tensor:
        return self.w_in

    def out_weight(self) -> torch.Tensor:
        return self.w_o

    def forward(self, x, step, cache):
        return self.forward_projected(ops.linear(x, self.w_in, self.ctx.dtype), step, cache)

    def forward_projected(self, row, step, cache):
        heads = torch.empty((step.n_tokens, self.heads_out), dtype=self.ctx.dtype, device=row.device)
        self.from_projection(row, step, cache, heads)
        return ops.linear(heads, self.w_o, self.ctx.dtype, parts_ok=True)

    def from_projection(self, row, step, cache, out):
        """`row` [n, in_rows] (the packed projection, possibly a column range) -> the normed, gated heads before the
        output product, written to `out` [n, inner] (possibly a column range)."""
        inner, gn, dt = self.inner, self.g * self.n, self.ctx.dtype
        state = cache.state
        mats = self.h * self.n * self.e
        conv_state = state[:, mats:] if self.taps > 1 else None
        xbc = ops.short_conv(row[:, inner:inner + self.conv_channels], self.conv_w, conv_state, step.cu_seqlens,
                             step.state_slots, step.n_entries, dt, bias=self.conv_b, act="silu")
        packed = ops.mamba_prepare(xbc, inner, inner + gn, row[:, 2 * inner + 2 * gn:2 * inner + 2 * gn + self.h],
                                   self.dt_bias, self.a_log, self.h, self.g, self.n)
        o = ops.state_scan(packed, xbc, 0, state, step.cu_seqlens, step.state_slots, step.n_entries, self.e)
        return ops.mamba_finish(o, xbc[:, :inner], row[:, :inner], self.skip, self.norm, out, self.h, self.e, self.ng,
                                self.spec.norm_eps)


register_mixer("state_space", StateSpace)
