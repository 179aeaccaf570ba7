"""A model put together from a `ModelSpec`: embedding, blocks in their run order, final
norm, output matrix (jllm/model/common.py:150-170).  It owns no cache and no batching: the
step hands it a `StepContext` and the per-layer cache views."""

from __future__ import annotations

import torch

from .. import ops
from .base import BuildContext, Part, TensorSpec
from .block import build_block
from .registry import NORMS, build


class Model(Part):
    def __init__(self, spec, ctx: BuildContext):
        spec.validate()
        self.spec, self.ctx = spec, ctx
        self.layers = [build_block(layer, ctx) for layer in spec.layers]
        self.final_norm = build(NORMS, "norm", spec.final_norm, "", ctx)
        self.embedding = self.lm_head = None
        # A cache belongs to a place in the run order, not to a layer: a layer that the order
        # names twice shares its weights between the two places but keeps keys and values
        # (or state) for each.  A layer with `cache_from` reads the cache of the latest
        # earlier place at which the layer it names ran.
        self.order = tuple(spec.run_order())
        self.reinject = frozenset(spec.reinject)
        self.position_table = self.pass_table = None
        self.pass_rows = dict(spec.pass_vectors[1]) if spec.pass_vectors is not None else {}
        self.place_cache = []
        self.place_names = [f"layer {i}" if self.order.count(i) == 1 else f"layer {i} (place {k})"
                            for k, i in enumerate(self.order)]
        for k, i in enumerate(self.order):
            src = spec.layers[i].cache_from
            if src is None:
                self.place_cache.append(k)
            else:
                self.place_cache.append(max(kk for kk in range(k) if self.order[kk] == src))

    # -------------------------------------------------------------------- weights
    def tensor_specs(self):
        s = self.spec
        out = {s.embedding_name: TensorSpec((s.vocab_size, s.hidden_size))}
        if s.position_table_name is not None:
            out[s.position_table_name] = TensorSpec((s.max_position, s.hidden_size))
        if s.pass_vectors is not None:
            rows = 1 + max(row for _, row in s.pass_vectors[1])
            out[s.pass_vectors[0]] = TensorSpec((rows, s.hidden_size), kind="vector", init="normal")
        for layer in self.layers:
            out.update(layer.tensor_specs())
        out.update(self.final_norm.tensor_specs())
        if s.lm_head_name is not None:
            out[s.lm_head_name] = TensorSpec((s.vocab_size, s.hidden_size))
        return out

    def optional_tensors(self):
        """Names that may be in the folder without being used (the output matrix of a tied
        model is ignored, jllm/model/weights.py:142-146)."""
        return ({"lm_head.weight"} if self.spec.lm_head_name is None else set()) | set(self.spec.unused_tensors)

    def bind(self, tensors):
        s = self.spec
        self.embedding = tensors[s.embedding_name].contiguous()
        if s.position_table_name is not None:
            self.position_table = tensors[s.position_table_name].contiguous()
        if s.pass_vectors is not None:
            self.pass_table = tensors[s.pass_vectors[0]].contiguous()
        for layer in self.layers:
            layer.bind(tensors)
        self.final_norm.bind(tensors)
        head = self.embedding if s.lm_head_name is None else tensors[s.lm_head_name]
        self.lm_head = self.compute_weight(head, self.ctx).contiguous()

    def kernels(self):
        names = {"embed", "norm", "gemm_simt"}
        names.update(getattr(self.final_norm, "kernels", ()))
        if self.pass_table is not None or self.spec.pass_vectors is not None:
            names.add("dyt")
        if self.spec.logit_softcap or self.spec.logit_scale is not None:
            names.add("activation")
        if self.ctx.dtype == torch.bfloat16:
            names.update(("linear_skinny", "linear_stream"))
        for layer in self.layers:
            names.update(layer.kernels)
            for part in layer.parts():
                names.update(part.kernels)
        return sorted(names)

    def capturable(self) -> bool:
        """Whether a step of this model may be captured into a CUDA graph and replayed: every part reads the
        batch from the device tensors of the step context only (`Part.capturable`)."""
        return all(getattr(part, "capturable", True) for layer in self.layers for part in layer.parts()) \
            and getattr(self.final_norm, "capturable", True)

    # ---------------------------------------------------------------------- cache
    def cache_needs(self):
        """Per place in the run order: what the layer there needs to keep, or None (nothing, or
        it reads another place's cache)."""
        def need(block):          # an arrangement that keeps something of its own says so; else it is the mixer's
            f = getattr(block, "cache_need", None)
            return f() if f is not None else block.mixer.cache_need()

        return [need(self.layers[i]) if self.place_cache[k] == k else None for k, i in enumerate(self.order)]

    def tile_classes(self, page_size: int):
        """The attention work lists that the mixers of this model want (see BatchBuilder)."""
        classes = set()
        for layer in self.layers:
            f = getattr(layer.mixer, "tile_classes", None)
            if f is not None:
                classes.update(tuple(c) for c in f(page_size))
        return sorted(classes)

    # ----------------------------------------------------------------------- step
    def forward(self, step, caches, tap=None) -> torch.Tensor:
        """Logits [n_logit_rows, vocab] float32 for one batch; caches are updated in place.  `tap(place, stream)`,
        if given, is called after every place of the run order with a copy of the stream as that layer leaves
        it (for comparing a model layer by layer; it costs a pass over the stream per layer)."""
        with ops.trace_range("embedding"):
            h = ops.embed_gather(self.embedding, step.token_ids)
            if self.position_table is not None:      # a learned vector per position (a position beyond the table sets the
                ops.embed_gather(self.position_table, step.positions, out=h, accumulate=True)   # status word)
        delta = None
        step.stream_copy = None
        for k, i in enumerate(self.order):
            if k in self.reinject:
                # the embedding output enters the stream again, after what the layer before left un-added
                if delta is not None:
                    ops.residual_add(h, delta)
                    delta = None
                step.stream_copy = None
                ops.embed_gather(self.embedding, step.token_ids, out=h, accumulate=True)
            if k in self.pass_rows:
                if delta is not None:
                    ops.residual_add(h, delta)
                    delta = None
                step.stream_copy = None
                ops.add_row(h, self.pass_table[self.pass_rows[k]])
            with ops.trace_range(self.place_names[k]):
                h, delta = self.layers[i].forward(h, delta, step, caches[self.place_cache[k]])
            if tap is not None:
                tap(k, h.clone() if delta is None else ops.residual_add(h.clone(), delta))
        if step.n_logit_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=h.device)
        with ops.trace_range("final_norm"):
            x = self.final_norm.gather(h, delta, step.logit_rows)
        with ops.trace_range("lm_head"):
            logits = ops.linear(x, self.lm_head, torch.float32)
            if self.spec.logit_scale is not None:
                ops.scale_(logits, self.spec.logit_scale)
            if self.spec.logit_softcap:
                ops.softcap_(logits, self.spec.logit_softcap)
            return logits
