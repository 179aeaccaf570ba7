"""Causal grouped-query attention over the paged cache whose options are data (`GeneralAttentionSpec`).

    row  = x @ [W_q; W_k; W_v; W_g]^T                    one product over the packed matrix
    q, k   whole-projection RMSNorm, query temperature, rotation of a leading part of every head;
           k, v -> cache (v = k as projected where the spec says so)      csrc/attn_prepare.cu, 32-bit
           or, head by head: RMSNorm with one weight vector shared by the heads, rotation in halves or interleaved
           pairs, values unit-normed and rotated by their own position      csrc/head_prepare.cu, 32-bit
    a    = sum_j w_ij v_j over the visible keys, w = softmax(cap(q.k * scale)) or sigmoid(q.k * scale + bias_h)
    o    = a, or a1 - lam * a2 for two score maps, unit-normed; times a sigmoid gate        csrc/attn_finish.cu
           with rotated values every head of a is first turned back by the query's position   csrc/head_prepare.cu
    y    = o @ W_o^T

Keys have `key_dim` elements a head and values `value_dim`; the value cache has its own shape.  With two score
maps the rows of W_q and W_k are re-ordered when the weights are bound, from head by head [map 1 | map 2] to all
heads' map 1 followed by all heads' map 2: the attention kernel then sees 2H query heads on 2G key heads with
the ordinary grouping (query head i on key head i // (H/G)), and key head g reads value head g % G.

The part also offers its two products to an arrangement that packs them with another part's
(`in_weight`, `from_projection`, `out_weight`): both then read the same normed input in one product and add
their outputs in one product over the concatenated inputs.
"""

from __future__ import annotations

import math

import torch

from .. import ops
from ..config.model_spec import AttentionSpec
from .attention import Attention
from .base import PagedKVNeed, Part, TensorSpec
from .registry import POSITIONS, build, register_mixer


def distance_buckets(buckets: int, saturate: int) -> list:
    """The row of a learned distance-bias table [buckets, heads] that serves the key `n` positions back, for n = 0 ..
    `saturate`: exact up to half the table, n itself; beyond, logarithmic steps, half + floor(ln(n / half) /
    ln(saturate / half) * (buckets - half)), capped at the last row, which every distance from `saturate` on shares."""
    half = buckets // 2
    if half < 1 or saturate <= half:
        raise ValueError(f"distance bias: {buckets} buckets need at least 2 rows and a largest distance beyond {half}")
    out = []
    for n in range(saturate + 1):
        if n < half:
            out.append(n)
        else:
            out.append(min(buckets - 1, half + int(math.floor(math.log(n / half) / math.log(saturate / half) * (buckets - half)))))
    return out


class GeneralAttention(Part):
    kernels = ("attn_prepare", "attn_simt", "attn_finish", "gemm_simt")
    FOREVER = 1 << 30

    def __init__(self, spec, prefix, ctx):
        self.spec, self.ctx = spec, ctx
        self.prefix = f"{prefix}.{spec.prefix}" if spec.prefix else prefix
        self.h, self.g, self.d, self.dv = spec.num_heads, spec.num_kv_heads, spec.key_dim, spec.value_dim
        if self.h < 1 or self.g < 1 or self.h % self.g:
            raise ValueError(f"{self.h} query heads are not a multiple of {self.g} key/value heads")
        if spec.weights not in ("softmax", "sigmoid"):
            raise ValueError(f"attention weights {spec.weights!r} are not built (softmax and sigmoid are)")
        if spec.gate not in (None, "head", "element"):
            raise ValueError(f"output gate {spec.gate!r} is not built (head and element are)")
        if spec.values_from_keys and self.dv != self.d:
            raise ValueError("values that are the keys have the keys' size")
        if spec.twin is not None and spec.weights != "softmax":
            raise ValueError("two score maps are built for softmax weights")
        self.maps = 2 if spec.twin is not None else 1
        self.hq, self.hk, self.hv = self.maps * self.h, self.maps * self.g, self.g     # as the kernels see them
        self.position = build(POSITIONS, "position encoding", spec.position, self.prefix, ctx) \
            if spec.position is not None else None
        if self.position is not None and self.position.dim > self.d:
            raise ValueError("rotary dim exceeds the key size")
        self.writes_cache = True
        self.mask = ops.mask_code(spec.window, spec.chunk)
        # heads prepared one by one (csrc/head_prepare.cu) where the layer asks for what only that kernel does
        interleaved = self.position is not None and getattr(self.position, "layout", "halves") == "interleaved"
        self.by_head = (spec.head_norm_eps is not None or spec.value_norm_eps is not None or spec.rotate_values
                        or interleaved)
        if self.by_head and (spec.whole_norm_eps is not None or spec.query_temperature is not None
                             or spec.values_from_keys or spec.twin is not None):
            raise ValueError("norms per head, normed or rotated values and interleaved pairs are built without a "
                             "whole-projection norm, a query temperature, values taken from keys and two score maps")
        self.interleaved = interleaved
        self.value_freq = None
        if spec.rotate_values:
            if self.position is None or self.dv % 2:
                raise ValueError("rotated values need a position encoding and an even value size")
            self.value_freq = self.position.frequencies(self.dv).to(ctx.device)
        if self.by_head:            # neither the whole-projection preparation nor (without a gate) the finishing kernel runs
            unused = ("attn_prepare",) + (("attn_finish",) if spec.gate is None else ())
            self.kernels = tuple(k for k in self.kernels if k not in unused) + ("head_prepare",)
        # Which attention kernel: once queries and keys are prepared, a mixer with one softmax map, no cap and
        # values shaped like its keys IS the plain grouped-query attention, and goes the way of that mixer (the
        # tcgen05 kernels for heads of 128, mma.sync for 16/32/64, in bfloat16).  Every other bfloat16 mixer with
        # sizes in steps of 16 takes the tensor-core kernel compiled for its pair of sizes; the rest, and 32-bit,
        # the CUDA-core kernel.
        # a temperature per head, a bias by distance and a sink are options of both of these
        self.extras = spec.head_temperature or spec.distance_bias is not None or spec.sink
        if self.extras and (spec.twin is not None or (spec.sink and spec.weights != "softmax")):
            raise ValueError("head temperature, distance bias and sink are built for one softmax map")
        plain = (spec.twin is None and spec.weights == "softmax" and not spec.score_cap and self.hv == self.hk
                 and self.dv == self.d and not self.extras)
        self.plain = self.general = None
        if plain and ops.attn_mma_supports(ctx.dtype, self.d):
            self.plain = Attention(AttentionSpec(spec.hidden_size, self.hq, self.hk, self.d, spec.scale, prefix="",
                                                 window=self.mask or None), self.prefix, ctx)
            self.kernels += tuple(k for k in self.plain.kernels if k not in self.kernels and k != "rope_kv")
        elif ops.attn_general_mma_supports(ctx.dtype, self.d, self.dv):
            self.general = ops.attn_general_mma_library(self.d, self.dv)
            self.kernels += (self.general,)
        # heads of 128 with sigmoid weights, or with a softmax that has a temperature per head, a bias by distance or a
        # sink: prompt portions that fill a 128-row tile go to the tcgen05 kernel
        self.big_tiles = (self.general is not None and not spec.score_cap and self.hv == self.hk and self.dv == self.d == 128
                          and spec.twin is None and (spec.weights == "sigmoid") != bool(self.extras))
        if self.big_tiles:
            self.kernels += ("attn_tcgen05",)
        self.w_in = self.w_o = self.q_norm = self.k_norm = self.bias = None
        self.head_scale = self.dist_bias = self.sink = None
        self.lam = 0.0
        # columns of the packed projection
        self.k_off = self.hq * self.d
        self.v_off = -1 if spec.values_from_keys else self.k_off + self.hk * self.d
        self.g_off = self.k_off + self.hk * self.d + (0 if spec.values_from_keys else self.hv * self.dv)
        self.g_rows = {None: 0, "head": self.h, "element": self.h * self.dv}[spec.gate]
        self.in_rows = self.g_off + self.g_rows
        self.heads_out = self.h * self.dv

    # -------------------------------------------------------------------- weights
    def _names(self):
        keys = ("q", "k", "v", "g", "o", "q_norm", "k_norm", "bias", "temp", "rel", "sink")
        return {k: f"{self.prefix}.{n}" for k, n in zip(keys, self.spec.names)}

    def tensor_specs(self):
        n, s = self._names(), self.spec
        specs = {n["q"]: TensorSpec((self.hq * self.d, s.hidden_size)),
                 n["k"]: TensorSpec((self.hk * self.d, s.hidden_size)),
                 n["o"]: TensorSpec((s.hidden_size, self.heads_out))}
        if not s.values_from_keys:
            specs[n["v"]] = TensorSpec((self.hv * self.dv, s.hidden_size))
        if s.gate is not None:
            specs[n["g"]] = TensorSpec((self.g_rows, s.hidden_size))
        if s.whole_norm_eps is not None:
            specs[n["q_norm"]] = TensorSpec((self.hq * self.d,), kind="vector", init="ones_normal")
            specs[n["k_norm"]] = TensorSpec((self.hk * self.d,), kind="vector", init="ones_normal")
        if s.head_norm_eps is not None:
            specs[n["q_norm"]] = TensorSpec((self.d,), kind="vector", init="ones_normal")
            specs[n["k_norm"]] = TensorSpec((self.d,), kind="vector", init="ones_normal")
        if s.score_bias:
            specs[n["bias"]] = TensorSpec((self.h,), kind="vector", init="normal")
        if s.twin is not None:
            for name in s.twin.names:
                specs[f"{self.prefix}.{name}"] = TensorSpec((self.d,), kind="vector", init="normal")
        if s.head_temperature:
            specs[n["temp"]] = TensorSpec((self.h,), kind="vector", init="ones_normal")
        if s.distance_bias is not None:
            rows = s.distance_bias[0]
            specs[n["rel"]] = TensorSpec((-1 if rows is None else int(rows), self.h), kind="vector", init="normal")
        if s.sink:
            specs[n["sink"]] = TensorSpec((self.h,), kind="vector", init="normal")
        return specs

    def _maps_first(self, w: torch.Tensor, heads: int) -> torch.Tensor:
        """Rows [head][map][d] -> [map][head][d]."""
        if self.maps == 1:
            return w
        return w.reshape(heads, self.maps, self.d, -1).transpose(0, 1).reshape(w.shape)

    def bind(self, tensors):
        n, s = self._names(), self.spec
        mats = [self._maps_first(tensors[n["q"]], self.h), self._maps_first(tensors[n["k"]], self.g)]
        if not s.values_from_keys:
            mats.append(tensors[n["v"]])
        if s.gate is not None:
            mats.append(tensors[n["g"]])
        mats = [self.compute_weight(m, self.ctx) for m in mats]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.to(torch.float32) for m in mats]
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.w_o = self.compute_weight(tensors[n["o"]], self.ctx).contiguous()
        if s.whole_norm_eps is not None or s.head_norm_eps is not None:
            self.q_norm, self.k_norm = tensors[n["q_norm"]].contiguous(), tensors[n["k_norm"]].contiguous()
            if self.q_norm.dtype != self.k_norm.dtype:
                self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()
        if s.score_bias:
            self.bias = tensors[n["bias"]].to(torch.float32).contiguous()
        if s.head_temperature:
            self.head_scale = tensors[n["temp"]].to(torch.float32).contiguous()
        if s.distance_bias is not None:
            # the table by head and distance, not by bucket: the kernels index a head's row with min(distance, last)
            rel = tensors[n["rel"]].to(torch.float32)
            rows = distance_buckets(rel.shape[0], int(s.distance_bias[1]))
            self.dist_bias = rel[torch.tensor(rows, device=rel.device)].t().contiguous()
        if s.sink:
            self.sink = tensors[n["sink"]].to(torch.float32).contiguous()
        if s.twin is not None:
            lq1, lk1, lq2, lk2 = (tensors[f"{self.prefix}.{name}"].double() for name in s.twin.names)
            self.lam = math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + float(s.twin.offset)

    # ---------------------------------------------------------------------- cache
    def cache_need(self):
        s = self.spec
        if self.hv == self.hk and self.dv == self.d:
            return PagedKVNeed(self.hk, self.d, s.window or None, chunk=s.chunk or None)
        return PagedKVNeed(self.hk, self.d, s.window or None, v_heads=self.hv, v_head_dim=self.dv, chunk=s.chunk or None)

    def tile_classes(self, page_size: int):
        if self.plain is not None:
            return self.plain.tile_classes(page_size)
        if self.general is not None:
            small = ops.attn_general_mma_tokens_per_tile(self.hq, self.hk)
            if self.big_tiles and ops.attn_tcgen05_supports(self.ctx.dtype, self.d, self.hq, self.hk, page_size, 0):
                big = ops.attn_tcgen05_tokens_per_tile(self.hq, self.hk)
                if big > small:
                    return [(small, 2, big), (big, big, self.FOREVER)]
            return [(small, 2, self.FOREVER)]
        return [(ops.attn_simt_tokens_per_tile(self.hq, self.hk), 2, self.FOREVER)]

    # ----------------------------------------------------------------------- step
    def in_weight(self) -> torch.Tensor:
        return self.w_in

    def out_weight(self) -> torch.Tensor:
        return self.w_o

    def forward(self, x, step, cache):
        dt = self.ctx.dtype
        row = ops.linear(x, self.w_in, dt)
        heads = torch.empty((step.n_tokens, self.heads_out), dtype=dt, device=x.device)
        self.from_projection(row, step, cache, heads)
        return ops.linear(heads, self.w_o, dt, parts_ok=True)

    def forward_projected(self, row, step, cache):
        """From the packed projection to the mixer's output, as one tensor."""
        heads = torch.empty((step.n_tokens, self.heads_out), dtype=self.ctx.dtype, device=row.device)
        self.from_projection(row, step, cache, heads)
        return ops.linear(heads, self.w_o, self.ctx.dtype)

    def from_projection(self, row, step, cache, out):
        """`row` [n, in_rows] (the packed projection, possibly a column range of a wider tensor) -> the heads
        before the output projection, written to `out` [n, heads * value_dim] (possibly a column range)."""
        s, dt, n = self.spec, self.ctx.dtype, step.n_tokens
        table = step.block_tables[cache.group]
        writes = self.writes_cache and cache.writes
        q = torch.empty((n, self.hq * self.d), dtype=dt, device=row.device)
        coef, every = s.query_temperature if s.query_temperature is not None else (0.0, 0)
        freq = self.position.table() if self.position is not None else None
        if self.by_head:
            ops.head_prepare(row, 0, self.k_off, self.v_off, q, step.positions, step.token_entry, table, freq,
                             self.interleaved, self.q_norm, self.k_norm, s.head_norm_eps or s.value_norm_eps or 0.0,
                             s.value_norm_eps is not None, self.value_freq, cache.k if writes else None,
                             cache.v if writes else None, self.hq, self.hk, self.hv, self.d, self.dv)
        else:
            ops.attn_prepare(row, 0, self.k_off, self.v_off, q, step.positions, step.token_entry, table, freq,
                             self.q_norm, self.k_norm, s.whole_norm_eps or 0.0, coef, every, cache.k if writes else None,
                             cache.v if writes else None, self.hq, self.hk, self.hv, self.d, self.dv)
        gate = row[:, self.g_off:self.g_off + self.g_rows] if s.gate is not None else None
        twin = s.twin
        if self.value_freq is not None and twin is None and gate is None:
            # the heads' outputs are turned back by the query's position, on the way to where they are wanted
            a = out if out.is_contiguous() else torch.empty((n, self.hq * self.dv), dtype=dt, device=row.device)
            self.attend(q, a, step, cache, table)
            return ops.head_rotate(a, step.positions, self.value_freq, self.interleaved, self.h, self.dv, sign=-1.0, out=out)
        if self.value_freq is not None:
            raise ValueError("rotated values with a gate or two score maps are not built")
        direct = twin is None and gate is None and out.is_contiguous()
        # two maps are subtracted in 32-bit: the attention kernel leaves them as floats
        a = out if direct else torch.empty((n, self.hq * self.dv), dtype=torch.float32 if twin is not None else dt,
                                           device=row.device)
        self.attend(q, a, step, cache, table)
        if not direct:
            ops.attn_finish(a, out, self.h, self.dv, maps=self.maps, lam=self.lam,
                            unit_norm_eps=None if twin is None else twin.eps,
                            post=1.0 if twin is None else 1.0 - twin.offset, gate=gate)
        return out

    def attend(self, q, a, step, cache, table):
        s = self.spec
        if self.plain is not None:
            return self.plain.attend(q, a, step, cache, table)
        common = (cache.k, cache.v, table, step.cu_seqlens, step.start_pos)
        extra = dict(score_cap=s.score_cap or 0.0, sigmoid=s.weights == "sigmoid", bias=self.bias)
        if self.extras:
            extra.update(head_scale=self.head_scale, dist_bias=self.dist_bias, sink=self.sink)
        if self.general is not None:
            def kernel(work, n_work, **split):
                ops.attn_general_mma(q, q.stride(0), a, *common, work, n_work, self.hq, self.hk, s.scale,
                                     window=self.mask, **split, **extra)
        else:
            def kernel(work, n_work, **split):
                ops.attn_simt(q, q.stride(0), a, *common, work, n_work, self.hq, self.hk, self.d, self.mask, s.scale,
                              v_dim=self.dv, **split, **extra)
        for cls in self.tile_classes(cache.k.shape[1]):
            work, n_work = step.tile_work[cls]
            if n_work and cls[1] > 2:                      # the class of whole 128-row tiles
                ops.attn_tcgen05(q, q.stride(0), a, *common, work, n_work, self.hq, self.hk, self.d, s.scale,
                                 sigmoid=s.weights == "sigmoid", bias=self.bias, head_scale=self.head_scale,
                                 dist_bias=self.dist_bias, sink=self.sink, window=self.mask)
            elif n_work:
                kernel(work, n_work)
        dwork, n_dec = step.decode_work
        if n_dec:
            split = self.ctx.decode_split_size
            kernel(dwork, n_dec, split_size=split, n_splits=max(1, -(-step.max_seq_len // split)))


register_mixer("general_attention", GeneralAttention)
