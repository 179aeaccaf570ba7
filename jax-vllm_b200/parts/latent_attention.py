"""Attention over a low-rank latent cache.

A token leaves in the cache ONE row [c | r]: c = RMSNorm(first `latent_dim` outputs of the
down-projection) and r = the rotated last `rot_dim` outputs, shared by all heads.  Head h's key
is [W_uk_h c | r] and its value W_uv_h c.  Neither is ever formed: since

    q_plain . (W_uk_h c) = (W_uk_h^T q_plain) . c        and        sum_j p_j W_uv_h c_j = W_uv_h (sum_j p_j c_j),

the step multiplies the plain part of every query head by W_uk_h^T, runs attention with ONE
key/value head whose key row is the cache row and whose value is the row's first
`latent_dim` elements, and multiplies each head's result by W_uv_h:

    row   = x @ [W_q; W_dkv; W_g]^T                       one product over the packed matrix
    q_lat = q_plain_h @ W_uk_h      per head              ops.bmm_heads
    cache row, q = [q_lat | rot(q_rot)]                   csrc/latent_prepare.cu (32-bit norm, angles, cos, sin)
    o_lat = softmax(q k^T * scale + causal mask) c        the paged attention kernels, keys and values one tensor
    o     = (o_lat_h @ W_uv_h^T) * sigmoid(gate)          ops.bmm_heads, ops.gate_heads
    y     = o @ W_o^T

A layer that reads another layer's cache has no down-projection and writes nothing.

Options (`LatentAttentionSpec`): queries through a latent of their own (row = x @ [W_dq; W_dkv; W_g]^T, c_q =
RMSNorm(first rows), q = c_q @ W_uq^T, a second product); a window of positions; a learned sink per head in the
softmax's denominator; interleaved pairs in the rotation (the position encoding's layout).
"""

from __future__ import annotations

import torch

from .. import ops
from .base import PagedKVNeed, Part, TensorSpec
from .registry import POSITIONS, build, register_mixer


class LatentAttention(Part):
    kernels = ("latent_prepare", "attn_simt", "gemm_simt")

    def __init__(self, spec, prefix, ctx):
        self.spec, self.ctx = spec, ctx
        self.prefix = f"{prefix}.{spec.prefix}" if spec.prefix else prefix
        self.h, self.dp, self.dr = spec.num_heads, spec.plain_dim, spec.rot_dim
        self.dv, self.dc = spec.value_dim, spec.latent_dim
        self.dk = self.dc + self.dr                     # a cache row, and a query head as the attention kernel sees it
        self.position = build(POSITIONS, "position encoding", spec.position, self.prefix, ctx) \
            if spec.position is not None else None
        if self.position is not None and self.position.dim != self.dr:
            raise ValueError("the rotated part of a head is rotated whole: the rotation's size must equal rot_dim")
        if self.dr % 2:
            raise ValueError("rot_dim must be even")
        self.interleaved = self.position is not None and getattr(self.position, "layout", "halves") == "interleaved"
        self.mask = ops.mask_code(spec.window, None)
        self.dq = spec.query_latent_dim
        self.sink = None
        self.writes_cache = True          # set False by the model for a layer that reads another's cache
        # bfloat16 with a row size the tensor-core kernels are built for; else the CUDA-core kernel
        # (the kernels built for fixed head sizes have no sink)
        self.use_mma = ops.attn_mma_supports(ctx.dtype, self.dk) and spec.sink is None
        # other row sizes in bfloat16: the tensor-core kernel written for latent rows (key = the row, value = its start)
        self.use_latent_mma = not self.use_mma and ops.attn_latent_mma_supports(ctx.dtype, self.dk, self.dc)
        if self.use_latent_mma:
            self.kernels = ("latent_prepare", "attn_latent_mma", "gemm_simt", "linear_skinny")
        if self.use_mma:
            self.kernels = ("latent_prepare", "attn_mma", "gemm_simt", "linear_skinny")
            if self.dk == 128:
                self.kernels += ("attn_tcgen05", "attn_decode_tcgen05")
        if self.dq is not None:
            self.kernels += ("head_prepare",)
        self.w_in = self.w_uk = self.w_uv = self.w_o = self.latent_norm = self.w_uq = self.q_norm = None

    # -------------------------------------------------------------------- weights
    def _names(self):
        keys = ("q", "dkv", "dkv_norm", "uk", "uv", "g", "o")
        return {k: f"{self.prefix}.{n}" for k, n in zip(keys, self.spec.names)}

    def tensor_specs(self):
        n, s = self._names(), self.spec
        qn = [f"{self.prefix}.{name}" for name in s.query_names]
        queries = {n["q"]: TensorSpec((self.h * (self.dp + self.dr), s.hidden_size))} if self.dq is None else \
            {qn[0]: TensorSpec((self.dq, s.hidden_size)), qn[1]: TensorSpec((self.dq,), kind="vector", init="ones_normal"),
             qn[2]: TensorSpec((self.h * (self.dp + self.dr), self.dq))}
        specs = {**queries,
                 n["uk"]: TensorSpec((self.h * self.dp, self.dc)),
                 n["uv"]: TensorSpec((self.h * self.dv, self.dc)),
                 n["o"]: TensorSpec((s.hidden_size, self.h * self.dv))}
        if s.output_gate:
            specs[n["g"]] = TensorSpec((self.h * self.dv, s.hidden_size))
        if s.sink is not None:
            specs[f"{self.prefix}.{s.sink}"] = TensorSpec((self.h,), kind="vector", init="normal")
        if self.writes_cache:
            specs[n["dkv"]] = TensorSpec((self.dc + self.dr, s.hidden_size))
            specs[n["dkv_norm"]] = TensorSpec((self.dc,), kind="vector", init="ones_normal")
        return specs

    def bind(self, tensors):
        n = self._names()
        qn = [f"{self.prefix}.{name}" for name in self.spec.query_names]
        mats = [tensors[n["q"] if self.dq is None else qn[0]]]
        if self.dq is not None:
            self.q_norm = tensors[qn[1]].contiguous()
            self.w_uq = self.compute_weight(tensors[qn[2]], self.ctx).contiguous()
        if self.spec.sink is not None:
            self.sink = tensors[f"{self.prefix}.{self.spec.sink}"].to(torch.float32).contiguous()
        self.kv_off = self.g_off = -1
        rows = mats[0].shape[0]
        if self.writes_cache:
            self.kv_off = rows
            mats.append(tensors[n["dkv"]])
            rows += mats[-1].shape[0]
            self.latent_norm = tensors[n["dkv_norm"]].contiguous()
        if self.spec.output_gate:
            self.g_off = rows
            mats.append(tensors[n["g"]])
        mats = [self.compute_weight(m, self.ctx) for m in mats]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.to(torch.float32) for m in mats]
        self.w_in = torch.cat(mats, dim=0).contiguous()
        # per head: W_uk_h^T [latent_dim, plain_dim] (the product is x @ W^T), W_uv_h [value_dim, latent_dim]
        uk = self.compute_weight(tensors[n["uk"]], self.ctx)
        self.w_uk = uk.reshape(self.h, self.dp, self.dc).transpose(1, 2).contiguous()
        self.w_uv = self.compute_weight(tensors[n["uv"]], self.ctx).reshape(self.h, self.dv, self.dc).contiguous()
        self.w_o = self.compute_weight(tensors[n["o"]], self.ctx).contiguous()

    # ---------------------------------------------------------------------- cache
    def cache_need(self):
        return PagedKVNeed(1, self.dk, self.spec.window or None, shared_kv=True)

    FOREVER = 1 << 30

    def _head_group(self) -> int:
        """The tcgen05 kernels take up to 16 query heads on one key/value head: more heads go through them in
        equal groups of the largest size up to 16 that divides their number (every group reads the same cache)."""
        return max(g for g in range(1, min(self.h, 16) + 1) if self.h % g == 0)

    def tile_classes(self, page_size: int):
        if self.use_latent_mma:
            return [(ops.attn_latent_mma_tokens_per_tile(self.h), 2, self.FOREVER)]
        small = (ops.attn_mma_tokens_per_tile if self.use_mma else ops.attn_simt_tokens_per_tile)(self.h, 1)
        g = self._head_group()
        if self.use_mma and ops.attn_tcgen05_supports(self.ctx.dtype, self.dk, g, 1, page_size, self.mask):
            big = ops.attn_tcgen05_tokens_per_tile(g, 1)
            if big > small:
                return [(small, 2, big), (big, big, self.FOREVER)]
            return [(big, 2, self.FOREVER)] if big == small else [(small, 2, self.FOREVER)]
        return [(small, 2, self.FOREVER)]

    # ----------------------------------------------------------------------- step
    def forward(self, x, step, cache):
        dt, n, H = self.ctx.dtype, step.n_tokens, self.h
        row = ops.linear(x, self.w_in, dt)
        table = step.block_tables[cache.group]
        writes = self.writes_cache and cache.writes
        wide = row.dtype != torch.float32 and self.w_uk.dtype == torch.float32    # 32-bit-stored weights in 16-bit mode
        kv_row = None
        if self.dq is not None:
            # the queries come from a normed latent of their own, by a second product; the down-projection stays behind
            kv_row = row
            row = ops.linear(ops.rms_rows(row[:, :self.dq], self.q_norm, self.spec.latent_norm_eps), self.w_uq, dt)
        q_plain = row[:, :H * (self.dp + self.dr)].view(n, H, self.dp + self.dr)[:, :, :self.dp].transpose(0, 1)
        q = torch.empty((n, H * self.dk), dtype=dt, device=x.device)
        if dt == torch.float32:
            # the batched product writes the latent part of every query head in place
            ops.bmm_heads(q_plain, self.w_uk, out=q.view(n, H, self.dk)[:, :, :self.dc].transpose(0, 1))
            q_lat = None
        else:
            q_lat = ops.bmm_heads(q_plain, self.w_uk.to(dt) if wide else self.w_uk)
        ops.latent_prepare(row, 0, self.kv_off, q_lat, q, step.positions, step.token_entry, table,
                           self.position.table() if self.position is not None else None,
                           self.latent_norm, self.spec.latent_norm_eps, cache.k if writes else None,
                           H, self.dp, self.dr, self.dc, kv_row=kv_row, interleaved=self.interleaved)
        o_lat = self.attend(q, step, cache, table)                      # [n, H, >= latent_dim], the latent part leads
        o = ops.bmm_heads(o_lat[:, :, :self.dc].transpose(0, 1), self.w_uv.to(dt) if wide else self.w_uv)
        gate = (row if kv_row is None else kv_row)[:, self.g_off:self.g_off + H * self.dv] if self.g_off >= 0 else None
        return ops.linear(ops.gate_heads(o, gate), self.w_o, dt, parts_ok=True)

    def attend(self, q, step, cache, table):
        """One key/value head: the cache row is the key, its leading latent part the value."""
        n, H, dk = step.n_tokens, self.h, self.dk
        common = (cache.k, cache.k, table, step.cu_seqlens, step.start_pos)
        if self.use_latent_mma:
            out = torch.empty((n, H * self.dc), dtype=q.dtype, device=q.device)
            args = (cache.k, table, step.cu_seqlens, step.start_pos)
            for cls in self.tile_classes(cache.k.shape[1]):
                work, n_work = step.tile_work[cls]
                ops.attn_latent_mma(q, q.stride(0), out, *args, work, n_work, H, dk, self.dc, self.spec.scale,
                                    window=self.mask, sink=self.sink)
            dwork, n_dec = step.decode_work
            if n_dec:
                # keys in splits of 32 to decode_split_size positions, so short that the blocks about fill the device
                # (one block a multiprocessor); the merge adds a request's splits in ascending order
                want = -(-step.max_seq_len * n_dec // ops.multiprocessors(q.device))
                split = min(self.ctx.decode_split_size, max(32, -(-want // 32) * 32))
                split = max(split, -(-step.max_seq_len // (32 * 1024)) * 32)        # the merge takes up to 1,024 splits
                ops.attn_latent_mma(q, q.stride(0), out, *args, dwork, n_dec, H, dk, self.dc, self.spec.scale,
                                    split_size=split, n_splits=max(1, -(-step.max_seq_len // split)),
                                    window=self.mask, sink=self.sink)
            return out.view(n, H, self.dc)
        if self.use_mma:
            # the tensor-core kernels take keys and values of one size: they return whole rows, the latent part leads
            out = torch.empty((n, H * dk), dtype=q.dtype, device=q.device)
            extra, per_head = {}, dk
            kernel = ops.attn_mma
        else:
            out = torch.empty((n, H * self.dc), dtype=q.dtype, device=q.device)
            extra, per_head = {"v_dim": self.dc, "sink": self.sink}, self.dc
            kernel = ops.attn_simt
        g = self._head_group()
        page = cache.k.shape[1]
        groups = [(q[:, i * dk:(i + g) * dk], out[:, i * dk:(i + g) * dk]) for i in range(0, H, g)] if self.use_mma else []
        big = ops.attn_tcgen05_tokens_per_tile(g, 1) \
            if self.use_mma and ops.attn_tcgen05_supports(self.ctx.dtype, dk, g, 1, page, self.mask) else 0
        for cls in self.tile_classes(page):
            work, n_work = step.tile_work[cls]
            if not n_work:
                continue
            if big and cls[0] == big:                      # whole tiles of the tcgen05 kernel, one head group at a time
                for qg, og in groups:
                    ops.attn_tcgen05(qg, q.stride(0), og, *common, work, n_work, g, 1, dk, self.spec.scale, window=self.mask)
            else:
                kernel(q, q.stride(0), out, *common, work, n_work, H, 1, dk, self.mask, self.spec.scale, **extra)
        dwork, n_dec = step.decode_work
        if n_dec and self.use_mma and ops.attn_decode_tcgen05_supports(self.ctx.dtype, dk, g, 1, page, self.mask, n_dec):
            for qg, og in groups:
                ops.attn_decode_tcgen05(qg, q.stride(0), og, *common, dwork, n_dec, g, 1, dk, self.spec.scale)
        elif n_dec:
            split = self.ctx.decode_split_size
            n_splits = max(1, -(-step.max_seq_len // split))
            kernel(q, q.stride(0), out, *common, dwork, n_dec, H, 1, dk, self.mask, self.spec.scale,
                   split_size=split, n_splits=n_splits, **extra)
        return out.view(n, H, per_head)


register_mixer("latent_attention", LatentAttention)
