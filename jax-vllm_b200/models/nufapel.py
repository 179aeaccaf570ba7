"""Nufapel: config.json -> typed configuration -> `ModelSpec`.

A decoder-only design whose layers are listed one by one in config.json (`layers`: each entry has `type`, the mixer's
sizes under `mixer`, and `mlp` or null).  What the design fixes is fixed here; every size and constant that config.json
carries is read from it, and sizes that only a tensor's shape gives (rows of the distance-bias table, rank of the
decay's projection) are left open until the weights are bound.  With dyt(x) = tanh(alpha x) * w + b:

    x  = embed[token] + pos[position]
    h  = dyt1(x);  x <- x + sigmoid(rg1 h + b) * mixer(h);     h = dyt2(x);  x <- x + sigmoid(rg2 h + b) * ff(h)
    `loop` = {start, stop, times}: layers start .. stop-1 run `times` times in a row with the same weights, every pass
    with caches and states of its own; right before pass t the vector `loop.step`[t] is added to every token
    logits = cap * tanh(head dyt_final(x) / cap),  cap = `logit_softcap`

mixers:

    "general_delta"   a matrix state per head under the generalized delta rule (parts/recurrent.py, `delta_rule`)
    "parallel"        two mixers side by side, each RMS-normed, half their sum (parts/mixer_pair.py):
                      left:  causal softmax attention without rotation, with a temperature per head, a learned bias by
                             bucketed distance, a sink in the denominator and a sigmoid gate per head
                      right: a matrix memory with exponential gates (parts/recurrent.py, `matrix_memory`)

feed-forwards: `dense` (down(gelu(up h)), exact gelu) or `moe` (routed experts with sigmoid scores, groups that score
as the sum of their two best, clamped gated experts).  Tensor names: `embed`, `pos`, `loop.step`, `l<i>.norm1|norm2`
(+ `.b`, `.alpha`), `l<i>.rg1|rg2` (+ `.b`), `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
"""

from __future__ import annotations

import copy
import json
from dataclasses import dataclass
from pathlib import Path

from ..config.model_spec import (DeltaRuleSpec, DenseMLPSpec, GeneralAttentionSpec, LayerSpec, MatrixMemorySpec,
                                 MixerPairSpec, ModelSpec, NormSpec, RoutedExpertsSpec)

ARCHITECTURE = "Nufapel"
MIXERS = ("general_delta", "parallel")
FEED_FORWARDS = ("dense", "moe")


def _need(d: dict, keys, where: str) -> None:
    if not isinstance(d, dict):
        raise KeyError(f"config.json: {where} is not an object")
    missing = [k for k in keys if k not in d]
    if missing:
        raise KeyError(f"config.json: {where} lacks {missing}")


def _positive(d: dict, keys, where: str) -> None:
    for k in keys:
        if int(d[k]) < 1:
            raise ValueError(f"{where}.{k} must be positive")


@dataclass(frozen=True)
class NufapelConfig:
    vocab: int
    width: int
    norm_eps: float
    max_positions: int
    logit_softcap: float | None
    layers: tuple                 # the entries of config.json's `layers`, as read
    loop: tuple | None            # (start, stop, times), or None: every layer runs once

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, c: dict) -> "NufapelConfig":
        _need(c, ("vocab", "width", "layers", "norm", "max_positions"), "the top level")
        _need(c["norm"], ("eps",), "norm")
        loop = c.get("loop")
        if loop is not None:
            _need(loop, ("start", "stop", "times"), "loop")
            loop = (int(loop["start"]), int(loop["stop"]), int(loop["times"]))
        cap = c.get("logit_softcap")
        cfg = cls(vocab=int(c["vocab"]), width=int(c["width"]), norm_eps=float(c["norm"]["eps"]),
                  max_positions=int(c["max_positions"]), logit_softcap=None if cap is None else float(cap),
                  layers=tuple(copy.deepcopy(layer) for layer in c["layers"]), loop=loop)
        cfg.validate()
        return cfg

    @classmethod
    def from_path(cls, path) -> "NufapelConfig":
        p = Path(path)
        if p.is_dir():
            p = p / "config.json"
        return cls.from_dict(json.loads(p.read_text()))

    def validate(self) -> None:
        if self.vocab < 1 or self.width < 1 or self.max_positions < 1 or not self.layers:
            raise ValueError("vocab, width, max_positions and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ValueError("norm.eps must be positive")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ValueError("logit_softcap must be positive")
        if self.loop is not None:
            a, b, times = self.loop
            if not 0 <= a < b <= len(self.layers) or times < 1:
                raise ValueError(f"loop {self.loop} does not fit {len(self.layers)} layers")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            kind, mx = layer["type"], layer["mixer"]
            if kind not in MIXERS:
                raise ValueError(f"{where}: mixer type {kind!r} is not part of this design ({MIXERS})")
            if kind == "general_delta":
                _need(mx, ("heads", "dim"), f"{where}.mixer")
                _positive(mx, ("heads", "dim"), f"{where}.mixer")
            else:
                _need(mx, ("left", "right"), f"{where}.mixer")
                left, right = mx["left"], mx["right"]
                _need(left, ("heads", "kv_heads", "dim", "vdim", "scale", "bias_max"), f"{where}.mixer.left")
                _positive(left, ("heads", "kv_heads", "dim", "vdim", "bias_max"), f"{where}.mixer.left")
                if int(left["heads"]) % int(left["kv_heads"]):
                    raise ValueError(f"{where}: heads must be a multiple of kv_heads")
                _need(right, ("heads", "dim", "vdim", "gate_cap"), f"{where}.mixer.right")
                _positive(right, ("heads", "dim", "vdim"), f"{where}.mixer.right")
                if not float(right["gate_cap"]) > 0:
                    raise ValueError(f"{where}: gate_cap must be positive")
            ml = layer.get("mlp")
            if ml is None:
                continue
            _need(ml, ("kind",), f"{where}.mlp")
            if ml["kind"] not in FEED_FORWARDS:
                raise ValueError(f"{where}: feed-forward kind {ml['kind']!r} is not part of this design ({FEED_FORWARDS})")
            if ml["kind"] == "dense":
                _need(ml, ("ff",), f"{where}.mlp")
                _positive(ml, ("ff",), f"{where}.mlp")
            else:
                _need(ml, ("expert", "router"), f"{where}.mlp")
                _need(ml["expert"], ("ff", "limit"), f"{where}.mlp.expert")
                ro = ml["router"]
                _need(ro, ("experts", "top", "groups", "scale"), f"{where}.mlp.router")
                _need(ro["groups"], ("count", "keep"), f"{where}.mlp.router.groups")
                E, top, n, keep = int(ro["experts"]), int(ro["top"]), int(ro["groups"]["count"]), int(ro["groups"]["keep"])
                if min(E, top, n, keep, int(ml["expert"]["ff"])) < 1 or E % n or keep > n or top > keep * (E // n):
                    raise ValueError(f"{where}: {E} experts, {n} groups, {keep} kept, top {top} do not fit")
                if not float(ml["expert"]["limit"]) > 0:
                    raise ValueError(f"{where}: the experts' limit must be positive")

    def to_dict(self) -> dict:
        """config.json content for this configuration."""
        d = {"architecture": ARCHITECTURE, "layers": [copy.deepcopy(layer) for layer in self.layers],
             "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width,
             "max_positions": self.max_positions}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.loop is not None:
            d["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        return d

    # ----------------------------------------------------------------- the model
    def run_order(self) -> tuple:
        """(the order in which the layers run, ((place, pass number), ...) for the places that start a pass)."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n)), ()
        a, b, times = self.loop
        order, starts = list(range(a)), []
        for t in range(times):
            starts.append((len(order), t))
            order += range(a, b)
        return tuple(order + list(range(b, n))), tuple(starts)

    def _mixer(self, kind: str, mx: dict):
        eps, W = self.norm_eps, self.width
        if kind == "general_delta":
            return DeltaRuleSpec(hidden_size=W, num_heads=int(mx["heads"]), head_dim=int(mx["dim"]), norm_eps=eps,
                                 decay_rank=int(mx["decay_rank"]) if "decay_rank" in mx else None, prefix="mix")
        left, right = mx["left"], mx["right"]
        buckets = int(left["buckets"]) if "buckets" in left else None
        attention = GeneralAttentionSpec(
            hidden_size=W, num_heads=int(left["heads"]), num_kv_heads=int(left["kv_heads"]), key_dim=int(left["dim"]),
            value_dim=int(left["vdim"]), scale=float(left["scale"]), gate="head", head_temperature=True,
            distance_bias=(buckets, int(left["bias_max"])), sink=True, prefix="left")
        memory = MatrixMemorySpec(hidden_size=W, num_heads=int(right["heads"]), key_dim=int(right["dim"]),
                                  value_dim=int(right["vdim"]), gate_cap=float(right["gate_cap"]), norm_eps=eps,
                                  prefix="right")
        return MixerPairSpec(hidden_size=W, left=attention, right=memory, eps=eps, coef=0.5, prefix="mix")

    def _feed_forward(self, ml):
        W = self.width
        if ml is None:
            return None
        if ml["kind"] == "dense":
            return DenseMLPSpec(hidden_size=W, intermediate_size=int(ml["ff"]), activation="gelu", prefix="mlp")
        ro, ex = ml["router"], ml["expert"]
        return RoutedExpertsSpec(hidden_size=W, num_experts=int(ro["experts"]), top_k=int(ro["top"]),
                                 expert_size=int(ex["ff"]), n_groups=int(ro["groups"]["count"]),
                                 keep_groups=int(ro["groups"]["keep"]), scoring="sigmoid", renormalize=True,
                                 activation="clamped_glu", group_score="top2_sum", renorm_eps=1e-20,
                                 weight_scale=float(ro["scale"]), limit=float(ex["limit"]), prefix="mlp")

    def to_spec(self) -> ModelSpec:
        eps, W = self.norm_eps, self.width
        layers = []
        for i, layer in enumerate(self.layers):
            ff = self._feed_forward(layer.get("mlp"))
            layers.append(LayerSpec(prefix=f"l{i}", mixer=self._mixer(layer["type"], layer["mixer"]), feed_forward=ff,
                                    mixer_norm=NormSpec(W, eps, "norm1", kind="dyt"),
                                    ffn_norm=None if ff is None else NormSpec(W, eps, "norm2", kind="dyt"),
                                    kind="pre_norm", residual_gates=("rg1", "rg2")))
        order, starts = self.run_order()
        # a layer without a feed-forward reads no second norm and no second gate, and a model without a loop no pass
        # vectors: a folder that holds them all the same is taken as it is
        unused = [f"l{i}.{name}" for i, layer in enumerate(layers) if layer.feed_forward is None
                  for name in ("norm2", "norm2.b", "norm2.alpha", "rg2", "rg2.b")]
        if not starts:
            unused.append("loop.step")
        spec = ModelSpec(architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=W, layers=tuple(layers),
                         final_norm=NormSpec(W, eps, "final.norm", kind="dyt"), embedding_name="embed",
                         lm_head_name="head", schedule=order, max_position=self.max_positions,
                         position_table_name="pos", pass_vectors=("loop.step", starts) if starts else None,
                         logit_softcap=self.logit_softcap, unused_tensors=tuple(unused))
        spec.validate()
        return spec
