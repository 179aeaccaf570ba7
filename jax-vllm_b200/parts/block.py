"""Arrangement of a layer: pre-norm with two residual sums
(jllm/model/common.py:140-147),

    h = h + mixer(norm1(h));  h = h + feed_forward(norm2(h)).

The stream `h` is float32 in every mode.  A block hands back its last branch output as
`delta`, not yet added, so that the next norm (of the next block, or the final one) adds
and normalises in one pass over the stream.  A branch output is a tensor [n, hidden] or an
`ops.PartialSum` (the parts of a product whose k was cut); the norms take either.
"""

from __future__ import annotations

import torch

from .. import ops
from ..ops import trace_range
from .base import FixedStateNeed, Part, TensorSpec
from .registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, TOKEN_INPUTS, build, register_block


class PreNormBlock(Part):
    """h = h + mixer(norm1(h));  h = h + feed_forward(norm2(h))   (the feed-forward is optional)

    With `residual_gates` each sublayer's result enters the stream through a gate, element by element:
    h = h + sigmoid(W_g x + b_g) * sublayer(x), x being the sublayer's input.  The gate's product reads the same x
    as the sublayer, so where the sublayer offers its input product (`in_weight`) the gate's matrix is stacked under
    it and one product serves both; the sum itself is made by the norm that follows (`ops.GatedDelta`).

    With `input_conv` = (taps, names) what each sublayer reads is u + conv(u), a short causal convolution over time on
    each channel of the normed stream (csrc/short_conv.cu; the norm hands u on in 32-bit and the sum is rounded to
    the compute type once).  The last taps - 1 rows of u are state of the sequence, for each sublayer: the block's
    cache need is then the mixer's followed by one `FixedStateNeed` a sublayer, and it gets a tuple of views."""

    def __init__(self, spec, prefix, ctx):
        p = spec.prefix
        self.spec, self.ctx = spec, ctx
        self.mixer_norm = build(NORMS, "norm", spec.mixer_norm, p, ctx)
        self.mixer = build(MIXERS, "mixer", spec.mixer, p, ctx)
        self.ffn_norm = self.feed_forward = None
        if spec.feed_forward is not None:
            self.ffn_norm = build(NORMS, "norm", spec.ffn_norm, p, ctx)
            self.feed_forward = build(FEED_FORWARDS, "feed-forward", spec.feed_forward, p, ctx)
        if spec.cache_from is not None:
            if not hasattr(self.mixer, "writes_cache"):
                raise ValueError(f"{p}: this mixer cannot read another layer's cache")
            self.mixer.writes_cache = False
        self.conv_taps, self.conv_names, self.conv_w = 0, (), [None, None]
        if spec.input_conv is not None:
            taps, names = spec.input_conv
            self.conv_taps = int(taps)
            if not 1 <= self.conv_taps <= ops.SHORT_CONV_MAX_TAPS:
                raise ValueError(f"{p}: an input convolution of {taps} taps is not built (1 .. {ops.SHORT_CONV_MAX_TAPS})")
            self.conv_names = tuple(f"{p}.{n}" for n in names)[:2 if spec.feed_forward is not None else 1]
            self.kernels = self.kernels + ("short_conv",)
        need = self.mixer.cache_need()
        self.mixer_views = len(need) if isinstance(need, (tuple, list)) else None     # None: one view, not a tuple
        gates = spec.residual_gates
        self.gate_names = None if gates is None else tuple(f"{p}.{g}" for g in gates)
        self.gate_w = [None, None]        # per sublayer: the gate's matrix alone, or None where it is stacked
        self.gate_b = [None, None]
        self.packed = [None, None]        # per sublayer: its input matrix with the gate's stacked under it
        if gates is not None:
            self.kernels = self.kernels + ("dyt", "gemm_simt")

    def parts(self):
        return tuple(part for part in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward) if part is not None)

    def tensor_specs(self):
        out = {}
        for part in self.parts():
            out.update(part.tensor_specs())
        if self.gate_names is not None:
            W = self.spec.mixer_norm.size
            for name in self.gate_names[:2 if self.feed_forward is not None else 1]:
                out[name] = TensorSpec((W, W))
                out[f"{name}.b"] = TensorSpec((W,), kind="vector", init="normal")
        for name in self.conv_names:
            out[name] = TensorSpec((self.spec.mixer_norm.size, self.conv_taps), kind="vector", init="normal")
        return out

    def cache_need(self):
        """What a place of the run order keeps for this layer: the mixer's need, and with an input convolution a
        state row of (taps - 1) x width 32-bit numbers for each sublayer behind it."""
        need = self.mixer.cache_need()
        if not self.conv_names or self.conv_taps < 2:
            return need
        own = tuple(FixedStateNeed(((self.conv_taps - 1) * self.spec.mixer_norm.size,), torch.float32) for _ in self.conv_names)
        return (tuple(need) if self.mixer_views is not None else (need,)) + own

    def _split_cache(self, cache):
        """(the mixer's cache view(s), the state views of the input convolutions)."""
        if not self.conv_names or self.conv_taps < 2:
            return cache, (None, None)
        k = self.mixer_views if self.mixer_views is not None else 1
        mixer = tuple(cache[:k]) if self.mixer_views is not None else cache[0]
        own = tuple(cache[k:]) + (None,)
        return mixer, own

    def _read(self, norm, i, h, delta, step, conv_state):
        """What sublayer i reads: the normed stream, with the input convolution added where the layer has one."""
        if not self.conv_names:
            return norm.norm(h, delta)
        u = norm.norm(h, delta, out_dtype=torch.float32)
        state = conv_state.state if conv_state is not None else None
        return ops.short_conv(u, self.conv_w[i], state, step.cu_seqlens, step.state_slots, step.n_entries, self.ctx.dtype,
                              residual=True)

    def bind(self, tensors):
        for part in self.parts():
            part.bind(tensors)
        for i, name in enumerate(self.conv_names):
            self.conv_w[i] = tensors[name].contiguous()
        if self.gate_names is None:
            return
        subs = (self.mixer, self.feed_forward)
        for i, sub in enumerate(subs):
            if sub is None:
                continue
            w = self.compute_weight(tensors[self.gate_names[i]], self.ctx).contiguous()
            self.gate_b[i] = tensors[f"{self.gate_names[i]}.b"].contiguous()
            self.gate_w[i], self.packed[i] = w, None
            ready = hasattr(sub, "forward_projected") if i == 0 else hasattr(sub, "from_projection")
            if ready and sub.in_weight().dtype == w.dtype:
                self.packed[i] = torch.cat([sub.in_weight(), w], dim=0).contiguous()

    def _mixer(self, x, step, cache):
        """The mixer's result, and the pre-activation of its gate (or None)."""
        dt = self.ctx.dtype
        if self.gate_names is None:
            return self.mixer.forward(x, step, cache), None
        if self.packed[0] is None:
            return _plain(self.mixer.forward(x, step, cache)), ops.linear(x, self.gate_w[0], dt)
        row = ops.linear(x, self.packed[0], dt)
        rm = self.mixer.in_rows
        return self.mixer.forward_projected(row[:, :rm], step, cache), row[:, rm:]

    def _feed_forward(self, x, step):
        dt = self.ctx.dtype
        ff = self.feed_forward
        if self.gate_names is None:
            return ff.forward(x, step), None
        if self.packed[1] is None:
            return _plain(ff.forward(x, step)), ops.linear(x, self.gate_w[1], dt)
        row = ops.linear(x, self.packed[1], dt)
        rm = ff.in_rows
        return ops.linear(ff.from_projection(row[:, :rm], step), ff.out_weight(), dt), row[:, rm:]

    def forward(self, h, delta, step, cache):
        step.stream_copy = None
        cache, conv_state = self._split_cache(cache)
        with trace_range("mixer_norm"):
            x = self._read(self.mixer_norm, 0, h, delta, step, conv_state[0])
        with trace_range("mixer"):
            a, z = self._mixer(x, step, cache)
            if z is not None:
                a = ops.GatedDelta(a, z, self.gate_b[0])
        if self.feed_forward is None:
            return h, a
        with trace_range("ffn_norm"):
            x = self._read(self.ffn_norm, 1, h, a, step, conv_state[1])
        with trace_range("feed_forward"):
            y, z = self._feed_forward(x, step)
            return h, (y if z is None else ops.GatedDelta(y, z, self.gate_b[1]))


def _plain(y):
    return y if isinstance(y, torch.Tensor) else y.tensor()


register_block("pre_norm", PreNormBlock)


class BranchNormBlock(Part):
    """A layer that norms every branch's OUTPUT before adding it, scaled, to the stream:

        h += m * norm1(mixer(h));  h += m * norm2(feed_forward(h));  h += m * norm_t(token_input(h, token))

    with m = `residual_scale`; the feed-forward and the token input are optional.  The branches read the stream
    itself, rounded to the compute type: each residual update (csrc/branch_norm.cu: norm, scale, sum and the
    rounded copy in one pass, 32-bit) hands the next branch its input.  Nothing is left un-added at the end, so
    the block takes a pending `delta` from an arrangement before it and returns none."""

    kernels = ("branch_norm",)

    def __init__(self, spec, prefix, ctx):
        p = spec.prefix
        self.spec, self.ctx = spec, ctx
        self.scale = float(spec.residual_scale)
        self.mixer_norm = build(NORMS, "norm", spec.mixer_norm, p, ctx)
        self.mixer = build(MIXERS, "mixer", spec.mixer, p, ctx)
        self.feed_forward = self.ffn_norm = self.token_input = None
        if spec.feed_forward is not None:
            self.ffn_norm = build(NORMS, "norm", spec.ffn_norm, p, ctx)
            self.feed_forward = build(FEED_FORWARDS, "feed-forward", spec.feed_forward, p, ctx)
        if spec.token_input is not None:
            self.token_input = build(TOKEN_INPUTS, "token input", spec.token_input, p, ctx)
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and not hasattr(norm, "weight"):
                raise ValueError(f"{p}: this arrangement needs norms with a plain weight")
        if spec.cache_from is not None:
            if not hasattr(self.mixer, "writes_cache"):
                raise ValueError(f"{p}: this mixer cannot read another layer's cache")
            self.mixer.writes_cache = False

    def parts(self):
        return tuple(part for part in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward, self.token_input)
                     if part is not None)

    def tensor_specs(self):
        out = {}
        for part in self.parts():
            out.update(part.tensor_specs())
        return out

    def bind(self, tensors):
        for part in self.parts():
            part.bind(tensors)

    def forward(self, h, delta, step, cache):
        dt = self.ctx.dtype
        # the stream rounded to the compute type, as the block before left it (only a block of this kind does)
        x, step.stream_copy = step.stream_copy, None
        if delta is not None:
            ops.residual_add(h, delta)
            x = None
        if x is None or dt == torch.float32:
            x = ops.cast_rows(h, dt)
        with trace_range("mixer"):
            a = self.mixer.forward(x, step, cache)
        with trace_range("mixer_norm"):
            x = self._add(h, a, self.mixer_norm.weight, self.mixer_norm.eps)
        if self.feed_forward is not None:
            with trace_range("feed_forward"):
                a = self.feed_forward.forward(x, step)
            with trace_range("ffn_norm"):
                x = self._add(h, a, self.ffn_norm.weight, self.ffn_norm.eps)
        if self.token_input is not None:
            with trace_range("token_input"):
                a = self.token_input.forward(x, step)
                x = self._add(h, a, self.token_input.norm_weight, self.token_input.eps)
        step.stream_copy = x if dt != torch.float32 else None
        return h, None

    def _add(self, h, branch, weight, eps):
        """The residual update; returns what the next branch reads (in 32-bit mode the stream itself)."""
        if self.ctx.dtype == torch.float32:
            ops.branch_norm_add(h, branch, weight, eps, self.scale)
            return h
        return ops.branch_norm_add(h, branch, weight, eps, self.scale, x_dtype=self.ctx.dtype)


register_block("branch_norm", BranchNormBlock)


class ParallelBlock(Part):
    """A layer whose two branches read ONE norm and are added together:

        u = norm(h);   h <- h + (mixer(u) + feed_forward(u))          (the feed-forward is optional)

    Where both parts offer their products (`in_weight`, `from_projection`, `out_weight`) and agree in type, the
    block runs two products a layer instead of four: u times the stacked input matrices [W_mixer_in; W_up], and
    the two parts' activations side by side times the output matrices joined along k, [W_o | W_down], whose sum
    over k IS mixer(u) + feed_forward(u).  The sum is handed on un-added, like every block's last branch."""

    def __init__(self, spec, prefix, ctx):
        p = spec.prefix
        self.spec, self.ctx = spec, ctx
        self.mixer_norm = build(NORMS, "norm", spec.mixer_norm, p, ctx)
        self.mixer = build(MIXERS, "mixer", spec.mixer, p, ctx)
        self.feed_forward = None if spec.feed_forward is None else \
            build(FEED_FORWARDS, "feed-forward", spec.feed_forward, p, ctx)
        if spec.cache_from is not None:
            if not hasattr(self.mixer, "writes_cache"):
                raise ValueError(f"{p}: this mixer cannot read another layer's cache")
            self.mixer.writes_cache = False
        self.w_in = self.w_out = None

    def parts(self):
        return tuple(part for part in (self.mixer_norm, self.mixer, self.feed_forward) if part is not None)

    def tensor_specs(self):
        out = {}
        for part in self.parts():
            out.update(part.tensor_specs())
        return out

    def bind(self, tensors):
        for part in self.parts():
            part.bind(tensors)
        both = [part for part in (self.mixer, self.feed_forward) if part is not None]
        self.w_in = self.w_out = None
        if all(hasattr(part, "from_projection") for part in both):
            ins, outs = [part.in_weight() for part in both], [part.out_weight() for part in both]
            if len({w.dtype for w in ins + outs}) == 1:
                self.w_in = torch.cat(ins, dim=0).contiguous() if len(ins) > 1 else ins[0]
                self.w_out = torch.cat(outs, dim=1).contiguous() if len(outs) > 1 else outs[0]

    def forward(self, h, delta, step, cache):
        step.stream_copy = None
        dt = self.ctx.dtype
        with trace_range("norm"):
            u = self.mixer_norm.norm(h, delta)
        if self.w_in is None:                       # parts without the packed interface: two branches, two sums
            with trace_range("mixer"):
                a = self.mixer.forward(u, step, cache)
            if self.feed_forward is None:
                return h, a
            ops.residual_add(h, a)
            with trace_range("feed_forward"):
                return h, self.feed_forward.forward(u, step)
        with trace_range("in"):
            row = ops.linear(u, self.w_in, dt)
        rm, km = self.mixer.in_rows, self.mixer.heads_out
        acts = torch.empty((step.n_tokens, self.w_out.shape[1]), dtype=dt, device=row.device)
        with trace_range("mixer"):
            self.mixer.from_projection(row[:, :rm], step, cache, acts[:, :km])
        if self.feed_forward is not None:
            with trace_range("feed_forward"):
                self.feed_forward.from_projection(row[:, rm:], step, acts[:, km:])
        with trace_range("out"):
            return h, ops.linear(acts, self.w_out, dt, parts_ok=True)


register_block("parallel", ParallelBlock)


def build_block(spec, ctx):
    return build(BLOCKS, "block", spec, spec.prefix, ctx)
