"""Mixers that keep a matrix per head and request instead of keys and values per token (csrc/recurrent.cu).

    delta_rule      S <- diag(w) S - (a u)(u^T S) + k v^T,  o = S^T r           (the generalized delta rule: both
                    terms read the old S; u the unit key; w a decay and a a removal rate per key channel)
    matrix_memory   S <- keep S + take k v^T, n <- keep n + take k, o = S^T q / (max(|n . q|, exp(-m)) + 1e-6)
                    with keep, take from a forget and an input gate in the log domain under a running maximum m

Both then divide each head's o by its root mean square, multiply by a weight and by sigmoid(W_g x), and project.
The state is float32 and lives in the request's state slot (`FixedStateNeed`): a portion of a prompt starts from what
the portion before left, a decoded token is a portion of one.  Everything that enters the recurrence besides the
projections is formed in 32-bit by the prepare kernels.  The parts offer their products to an arrangement that packs
them (`in_weight`, `from_projection`, `out_weight`).
"""

from __future__ import annotations

import torch

from .. import ops
from .base import FixedStateNeed, Part, TensorSpec
from .registry import register_mixer


class _StateMixer(Part):
    kernels = ("recurrent", "gemm_simt")

    def _bind_in(self, tensors, keys):
        mats = [self.compute_weight(tensors[self.names[k]], self.ctx) for k in keys]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.to(torch.float32) for m in mats]
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.w_o = self.compute_weight(tensors[self.names["o"]], self.ctx).contiguous()

    def in_weight(self) -> torch.Tensor:
        return self.w_in

    def out_weight(self) -> torch.Tensor:
        return self.w_o

    def forward_projected(self, row, step, cache):
        heads = torch.empty((step.n_tokens, self.heads_out), dtype=self.ctx.dtype, device=row.device)
        self.from_projection(row, step, cache, heads)
        return ops.linear(heads, self.w_o, self.ctx.dtype)

    def forward(self, x, step, cache):
        return self.forward_projected(ops.linear(x, self.w_in, self.ctx.dtype), step, cache)


class DeltaRule(_StateMixer):
    def __init__(self, spec, prefix, ctx):
        self.spec, self.ctx = spec, ctx
        self.prefix = f"{prefix}.{spec.prefix}" if spec.prefix else prefix
        self.h, self.d = int(spec.num_heads), int(spec.head_dim)
        if self.h < 1 or not 1 <= self.d <= ops.SCAN_MAX_KEY:
            raise ValueError(f"delta rule: heads of {self.d} are not built (1 .. {ops.SCAN_MAX_KEY})")
        keys = ("r", "k", "v", "g", "a", "a_b", "w1", "w2", "w0", "norm", "o")
        self.names = {k: f"{self.prefix}.{n}" for k, n in zip(keys, spec.names)}
        self.hd = self.h * self.d
        self.rank = spec.decay_rank
        self.heads_out = self.hd
        self.in_rows = None if self.rank is None else 5 * self.hd + self.rank
        self.w_in = self.w_o = self.w_up = self.a_bias = self.w_bias = self.norm = None

    def tensor_specs(self):
        n, W, hd = self.names, self.spec.hidden_size, self.hd
        rank = -1 if self.rank is None else self.rank
        out = {n[k]: TensorSpec((hd, W)) for k in ("r", "k", "v", "g", "a")}
        out.update({n["w1"]: TensorSpec((rank, W)), n["w2"]: TensorSpec((hd, rank)), n["o"]: TensorSpec((W, hd)),
                    n["a_b"]: TensorSpec((hd,), kind="vector", init="normal"),
                    n["w0"]: TensorSpec((hd,), kind="vector", init="normal"),
                    n["norm"]: TensorSpec((hd,), kind="vector", init="ones_normal")})
        return out

    def bind(self, tensors):
        n = self.names
        self.rank = int(tensors[n["w1"]].shape[0])
        if tensors[n["w2"]].shape[1] != self.rank:
            raise ValueError(f"{self.prefix}: the decay's two matrices differ in rank")
        self.in_rows = 5 * self.hd + self.rank
        self._bind_in(tensors, ("r", "k", "v", "g", "a", "w1"))
        self.w_up = self.compute_weight(tensors[n["w2"]], self.ctx).contiguous()
        self.a_bias = tensors[n["a_b"]].contiguous()
        self.w_bias = tensors[n["w0"]].to(self.a_bias.dtype).contiguous()
        self.norm = tensors[n["norm"]].contiguous()

    def cache_need(self):
        return FixedStateNeed((self.hd * self.d,), torch.float32)

    def from_projection(self, row, step, cache, out):
        hd, dt = self.hd, self.ctx.dtype
        low = ops.unary_act(row[:, 5 * hd:5 * hd + self.rank], "tanh")
        zw = ops.linear(low, self.w_up, dt)
        packed = ops.delta_prepare(row, 0, hd, 4 * hd, zw, self.a_bias, self.w_bias, self.h, self.d)
        o = ops.state_scan(packed, row, 2 * hd, cache.state, step.cu_seqlens, step.state_slots, step.n_entries, self.d)
        return ops.head_norm_gate(o, self.norm, row[:, 3 * hd:4 * hd], out, self.h, self.d, self.spec.norm_eps)


register_mixer("delta_rule", DeltaRule)


class MatrixMemory(_StateMixer):
    def __init__(self, spec, prefix, ctx):
        self.spec, self.ctx = spec, ctx
        self.prefix = f"{prefix}.{spec.prefix}" if spec.prefix else prefix
        self.h, self.d, self.dv = int(spec.num_heads), int(spec.key_dim), int(spec.value_dim)
        if self.h < 1 or not 1 <= self.d <= ops.SCAN_MAX_KEY or self.dv < 1:
            raise ValueError(f"matrix memory: keys of {self.d} are not built (1 .. {ops.SCAN_MAX_KEY})")
        if not spec.gate_cap > 0:
            raise ValueError("matrix memory: the gates' cap must be positive")
        keys = ("q", "k", "v", "g", "i", "i_b", "f", "f_b", "norm", "o")
        self.names = {k: f"{self.prefix}.{n}" for k, n in zip(keys, spec.names)}
        self.hd, self.hv = self.h * self.d, self.h * self.dv
        self.heads_out = self.hv
        self.in_rows = 2 * self.hd + 2 * self.hv + 2 * self.h
        self.w_in = self.w_o = self.i_bias = self.f_bias = self.norm = None

    def tensor_specs(self):
        n, W = self.names, self.spec.hidden_size
        return {n["q"]: TensorSpec((self.hd, W)), n["k"]: TensorSpec((self.hd, W)), n["v"]: TensorSpec((self.hv, W)),
                n["g"]: TensorSpec((self.hv, W)), n["i"]: TensorSpec((self.h, W)), n["f"]: TensorSpec((self.h, W)),
                n["i_b"]: TensorSpec((self.h,), kind="vector", init="normal"),
                n["f_b"]: TensorSpec((self.h,), kind="vector", init="normal"),
                n["norm"]: TensorSpec((self.hv,), kind="vector", init="ones_normal"), n["o"]: TensorSpec((W, self.hv))}

    def bind(self, tensors):
        n = self.names
        self._bind_in(tensors, ("q", "k", "v", "g", "i", "f"))
        self.i_bias = tensors[n["i_b"]].contiguous()
        self.f_bias = tensors[n["f_b"]].to(self.i_bias.dtype).contiguous()
        self.norm = tensors[n["norm"]].contiguous()

    def cache_need(self):
        # one row per request: the matrices of all heads, then their normalisers, then their running maxima
        return FixedStateNeed((self.hd * self.dv + self.hd + self.h,), torch.float32)

    def from_projection(self, row, step, cache, out):
        hd, hv, h = self.hd, self.hv, self.h
        state = cache.state
        mats = hd * self.dv
        packed, gates = ops.memory_gates(row, 0, hd, 2 * hd + 2 * hv, 2 * hd + 2 * hv + h, self.i_bias, self.f_bias,
                                         self.spec.gate_cap, self.d ** -0.5, state[:, mats + hd:], step.cu_seqlens,
                                         step.state_slots, step.n_entries, h, self.d)
        o = ops.state_scan(packed, row, 2 * hd, state, step.cu_seqlens, step.state_slots, step.n_entries, self.dv,
                           state_n=state[:, mats:mats + hd], gates=gates)
        return ops.head_norm_gate(o, self.norm, row[:, 2 * hd + hv:2 * hd + 2 * hv], out, h, self.dv, self.spec.norm_eps,
                                  gates=gates)


register_mixer("matrix_memory", MatrixMemory)
