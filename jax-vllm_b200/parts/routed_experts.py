"""A mixture of small feed-forward experts, each down(act(up(x))), no biases; or, with the activation
"clamped_glu", experts with a gate matrix: g = min(W_gate x, limit), u = clamp(W_up x, -limit, limit),
down(g * sigmoid(1.702 g) * (u + 1)) (the two matrices are stacked, the activation is a kernel of its own).

    z        = x @ W_router^T           32-bit accumulation and result (ops.linear)
    ids, w   = route(z)                 softmax scores in 32-bit, group-limited choice of the top_k (csrc/moe_route.cu)
    order    = pairs sorted by expert   every expert's rows padded to a row tile (csrc/moe_route.cu, jv_moe_align)
    a        = act(x[token] @ W_up_e^T) grouped product, rows gathered as they are read, activation in its epilogue
    y        = a @ W_down_e^T           grouped product
    out[t]   = sum_k w[t, k] * y[pos(t, k)]     added up in 32-bit, k ascending, by the reader of the result

The result is handed on as an `ops.PickedRows` (rows of y, which to pick and with which weight): the norm that
follows adds them up as it reads them.  The expert matrices are kept stacked, [experts, out, in].
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, TensorSpec
from .registry import register_feed_forward


class RoutedExperts(Part):
    kernels = ("moe_route", "moe_gemm_simt", "gemm_simt")

    def __init__(self, spec, prefix, ctx):
        if spec.activation not in ("gelu", "clamped_glu"):
            raise ValueError(f"routed experts: activation {spec.activation!r} is not built (gelu and clamped_glu are)")
        if spec.scoring not in ops.ROUTER_SCORINGS or spec.group_score not in ops.GROUP_SCORES:
            raise ValueError(f"routed experts: scoring {spec.scoring!r} with group score {spec.group_score!r} is not "
                             f"built ({', '.join(ops.ROUTER_SCORINGS)}; {', '.join(ops.GROUP_SCORES)})")
        self.gated = spec.activation == "clamped_glu"
        if self.gated and not spec.limit > 0:
            raise ValueError("routed experts: the clamped activation needs a positive limit")
        if self.gated:
            self.kernels = ("moe_route", "moe_gemm_simt", "gemm_simt", "activation")
        E, n, keep = spec.num_experts, spec.n_groups, spec.keep_groups
        if E % n or not 1 <= keep <= n or not 1 <= spec.top_k <= keep * (E // n):
            raise ValueError(f"routed experts: {E} experts, {n} groups, {keep} kept, top {spec.top_k} do not fit")
        self.spec, self.ctx = spec, ctx
        self.prefix = f"{prefix}.{spec.prefix}" if spec.prefix else prefix
        self.w_router = self.w_up = self.w_down = None

    def tensor_specs(self):
        p, s = self.prefix, self.spec
        out = {f"{p}.router": TensorSpec((s.num_experts, s.hidden_size))}
        for e in range(s.num_experts):
            if self.gated:
                out[f"{p}.e{e}.gate"] = TensorSpec((s.expert_size, s.hidden_size))
            out[f"{p}.e{e}.up"] = TensorSpec((s.expert_size, s.hidden_size))
            out[f"{p}.e{e}.down"] = TensorSpec((s.hidden_size, s.expert_size))
        return out

    def bind(self, tensors):
        p, s = self.prefix, self.spec
        self.w_router = self.compute_weight(tensors[f"{p}.router"], self.ctx).contiguous()
        ups = [self.compute_weight(tensors[f"{p}.e{e}.up"], self.ctx) for e in range(s.num_experts)]
        if self.gated:      # [gate; up] of an expert stacked: one grouped product makes both
            gates = [self.compute_weight(tensors[f"{p}.e{e}.gate"], self.ctx) for e in range(s.num_experts)]
            if len({m.dtype for m in ups + gates}) > 1:
                ups, gates = [m.float() for m in ups], [m.float() for m in gates]
            ups = [torch.cat([g, u], dim=0) for g, u in zip(gates, ups)]
        downs = [self.compute_weight(tensors[f"{p}.e{e}.down"], self.ctx) for e in range(s.num_experts)]
        if len({m.dtype for m in ups + downs}) > 1:
            ups, downs = [m.float() for m in ups], [m.float() for m in downs]
        self.w_up = torch.stack(ups).contiguous()
        self.w_down = torch.stack(downs).contiguous()
        if self._tensor_cores():
            self.kernels = ("moe_route", "gemm_tcgen05", "gemm_simt") + (("activation",) if self.gated else ())

    # The grouped tcgen05 product works on 128-row tiles of 256 columns: it is taken for bfloat16 experts whose inner
    # sizes it can address (multiples of 8) and whose matrices are at least this wide; smaller ones, and the 32-bit
    # path, go to the CUDA-core product with its 32-row tiles.
    TCGEN05_MIN_SIZE = 128

    def _tensor_cores(self) -> bool:
        s = self.spec
        return (ops.moe_gemm_tcgen05_supports(self.ctx.dtype, self.w_up) and ops.moe_gemm_tcgen05_supports(self.ctx.dtype, self.w_down)
                and min(s.expert_size, s.hidden_size) >= self.TCGEN05_MIN_SIZE)

    def forward(self, x, step):
        s, dt = self.spec, self.ctx.dtype
        logits = ops.linear(x, self.w_router, torch.float32)       # 32-bit accumulation, 32-bit result
        ids, weights = ops.moe_route(logits, s.top_k, s.n_groups, s.keep_groups, s.renormalize, s.scoring, s.group_score,
                                     s.renorm_eps, s.weight_scale)
        first = None if self.gated else "gelu"
        if self._tensor_cores():
            _, pos_of, tile_expert, used = ops.moe_align(ids, s.num_experts, ops.MOE_TCGEN05_TILE)
            rows = ops.moe_gather_rows(x, pos_of, tile_expert.numel() * ops.MOE_TCGEN05_TILE)
            act = ops.moe_gemm_tcgen05(rows, self.w_up, tile_expert, act=first, used_tiles=used)
            if self.gated:
                act = ops.glu_clamped(act, s.limit)
            return ops.PickedRows(ops.moe_gemm_tcgen05(act, self.w_down, tile_expert, used_tiles=used), pos_of, weights)
        sorted_token, pos_of, tile_expert, _ = ops.moe_align(ids, s.num_experts, ops.moe_gemm_simt_tile())
        act = ops.moe_gemm_simt(x, sorted_token, self.w_up, tile_expert, dt, act=first)
        if self.gated:
            act = ops.glu_clamped(act, s.limit)
        y = ops.moe_gemm_simt(act, None, self.w_down, tile_expert, dt)
        return ops.PickedRows(y, pos_of, weights)


register_feed_forward("routed_experts", RoutedExperts)
