"""Gogivik: config.json -> typed configuration -> `ModelSpec`.

A decoder-only design whose layers are listed one by one in config.json (`layers`: each entry has `type`, the mixer's
sizes under `mixer`, and `mlp` or null).  What the design fixes is fixed here; every size and constant that config.json
carries is read from it.  With norm(x) = x / sqrt(mean(x^2) + eps) * (1 + w) and tapconv a causal convolution over
time on each channel (`canon.taps` taps, the last one on the current token):

    x = embed[token]
    u = norm1(x);  u <- u + tapconv1(u);  x <- x + mixer(u)
    u = norm2(x);  u <- u + tapconv2(u);  x <- x + down(relu(up u)^2)          (a layer may have no feed-forward)
    logits = head norm_final(x) * logit_scale

mixers:

    "attention"         grouped-query softmax attention (parts/general_attention.py): queries and keys RMS-normed per
                        head with one shared weight, rotated in halves over `rot.dims` elements with frequencies
                        divided by `rot.scaling.factor`; values unit-normed per head and rotated by their own position
                        over their whole size, the output turned back by the query's position; a query sees the earlier
                        positions of its chunk of `mask.size`
    "latent_attention"  keys and values from one normed latent a token plus one rotated key part shared by the heads,
                        queries from a normed latent of their own (parts/latent_attention.py); interleaved pairs; a
                        window of `mask.size` positions; a sink per head in the softmax's denominator
    "mamba2"            a state-space mixer with a short convolution (parts/state_space.py)

Tensor names: `embed`, `l<i>.norm1|norm2`, `l<i>.canon1|canon2`, `l<i>.mix.*`, `l<i>.mlp.up|down`, `final.norm`, `head`.
"""

from __future__ import annotations

import copy
import json
from dataclasses import dataclass
from pathlib import Path

from ..config.model_spec import (DenseMLPSpec, GeneralAttentionSpec, LatentAttentionSpec, LayerSpec, ModelSpec, NormSpec,
                                 RopeSpec, StateSpaceSpec)

ARCHITECTURE = "Gogivik"
MIXERS = ("attention", "latent_attention", "mamba2")
FEED_FORWARDS = ("dense",)


def _need(d, keys, where: str) -> None:
    if not isinstance(d, dict):
        raise KeyError(f"config.json: {where} is not an object")
    missing = [k for k in keys if k not in d]
    if missing:
        raise KeyError(f"config.json: {where} lacks {missing}")


def _positive(d: dict, keys, where: str) -> None:
    for k in keys:
        if int(d[k]) < 1:
            raise ValueError(f"{where}.{k} must be positive")


def _mask(mx: dict, where: str):
    m = mx.get("mask")
    if m is None:
        return None
    _need(m, ("size",), f"{where}.mask")
    if int(m["size"]) < 1:
        raise ValueError(f"{where}.mask.size must be positive")
    return int(m["size"])


def _rot(mx: dict, where: str, limit: int):
    """(base, dims, scaling factor) of a mixer's rotation, or None."""
    r = mx.get("rot")
    if r is None:
        return None
    _need(r, ("base", "dims"), f"{where}.rot")
    dims, factor = int(r["dims"]), 1.0
    if dims < 2 or dims % 2 or dims > limit:
        raise ValueError(f"{where}.rot.dims must be even, from 2 to {limit}")
    if not float(r["base"]) > 0:
        raise ValueError(f"{where}.rot.base must be positive")
    if r.get("scaling") is not None:
        _need(r["scaling"], ("factor",), f"{where}.rot.scaling")
        factor = float(r["scaling"]["factor"])
        if not factor > 0:
            raise ValueError(f"{where}.rot.scaling.factor must be positive")
    return float(r["base"]), dims, factor


@dataclass(frozen=True)
class GogivikConfig:
    vocab: int
    width: int
    norm_eps: float
    conv_taps: int | None         # taps of the convolution on what each sublayer reads; None: no such convolution
    logit_scale: float | None
    layers: tuple                 # the entries of config.json's `layers`, as read

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, c: dict) -> "GogivikConfig":
        _need(c, ("vocab", "width", "layers", "norm"), "the top level")
        _need(c["norm"], ("eps",), "norm")
        taps = None
        if c.get("canon") is not None:
            _need(c["canon"], ("taps",), "canon")
            taps = int(c["canon"]["taps"])
        scale = c.get("logit_scale")
        cfg = cls(vocab=int(c["vocab"]), width=int(c["width"]), norm_eps=float(c["norm"]["eps"]), conv_taps=taps,
                  logit_scale=None if scale is None else float(scale),
                  layers=tuple(copy.deepcopy(layer) for layer in c["layers"]))
        cfg.validate()
        return cfg

    @classmethod
    def from_path(cls, path) -> "GogivikConfig":
        p = Path(path)
        if p.is_dir():
            p = p / "config.json"
        return cls.from_dict(json.loads(p.read_text()))

    def validate(self) -> None:
        if self.vocab < 1 or self.width < 1 or not self.layers:
            raise ValueError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ValueError("norm.eps must be positive")
        if self.conv_taps is not None and not 1 <= self.conv_taps <= 8:
            raise ValueError("canon.taps must be from 1 to 8")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            kind, mx = layer["type"], layer["mixer"]
            if kind not in MIXERS:
                raise ValueError(f"{where}: mixer type {kind!r} is not part of this design ({MIXERS})")
            w = f"{where}.mixer"
            if kind == "attention":
                _need(mx, ("heads", "kv_heads", "dim", "vdim", "scale"), w)
                _positive(mx, ("heads", "kv_heads", "dim", "vdim"), w)
                if int(mx["heads"]) % int(mx["kv_heads"]):
                    raise ValueError(f"{where}: heads must be a multiple of kv_heads")
                if _rot(mx, w, int(mx["dim"])) is not None and int(mx["vdim"]) % 2:
                    raise ValueError(f"{where}: rotated values need an even vdim")
                _mask(mx, w)
            elif kind == "latent_attention":
                _need(mx, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale"), w)
                _positive(mx, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"), w)
                rot = _rot(mx, w, int(mx["rot_dim"]))
                if rot is not None and rot[1] != int(mx["rot_dim"]):
                    raise ValueError(f"{where}: the rotated part is rotated whole (rot.dims = rot_dim)")
                if int(mx["rot_dim"]) % 2:
                    raise ValueError(f"{where}: rot_dim must be even")
                _mask(mx, w)
            else:
                _need(mx, ("heads", "vdim", "state", "groups", "norm_groups", "conv"), w)
                _positive(mx, ("heads", "vdim", "state", "groups", "norm_groups", "conv"), w)
                if int(mx["heads"]) % int(mx["groups"]) or (int(mx["heads"]) * int(mx["vdim"])) % int(mx["norm_groups"]):
                    raise ValueError(f"{where}: heads must be a multiple of groups, and heads * vdim of norm_groups")
                if int(mx["conv"]) > 8:
                    raise ValueError(f"{where}: a convolution of more than 8 taps is not built")
            ml = layer.get("mlp")
            if ml is None:
                continue
            _need(ml, ("kind",), f"{where}.mlp")
            if ml["kind"] not in FEED_FORWARDS:
                raise ValueError(f"{where}: feed-forward kind {ml['kind']!r} is not part of this design ({FEED_FORWARDS})")
            _need(ml, ("ff",), f"{where}.mlp")
            _positive(ml, ("ff",), f"{where}.mlp")

    def to_dict(self) -> dict:
        """config.json content for this configuration."""
        d = {"architecture": ARCHITECTURE, "layers": [copy.deepcopy(layer) for layer in self.layers],
             "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.conv_taps is not None:
            d["canon"] = {"taps": self.conv_taps}
        if self.logit_scale is not None:
            d["logit_scale"] = self.logit_scale
        return d

    # ----------------------------------------------------------------- the model
    def _mixer(self, kind: str, mx: dict, where: str):
        eps, W = self.norm_eps, self.width
        if kind == "attention":
            rot = _rot(mx, where, int(mx["dim"]))
            position = None if rot is None else RopeSpec(dim=rot[1], theta=rot[0], exact_table=True, scaling_factor=rot[2],
                                                         layout="halves")
            return GeneralAttentionSpec(
                hidden_size=W, num_heads=int(mx["heads"]), num_kv_heads=int(mx["kv_heads"]), key_dim=int(mx["dim"]),
                value_dim=int(mx["vdim"]), scale=float(mx["scale"]), position=position, head_norm_eps=eps,
                value_norm_eps=eps, rotate_values=position is not None, chunk=_mask(mx, where), prefix="mix")
        if kind == "latent_attention":
            rot = _rot(mx, where, int(mx["rot_dim"]))
            position = None if rot is None else RopeSpec(dim=rot[1], theta=rot[0], exact_table=True, scaling_factor=rot[2],
                                                         layout="interleaved")
            return LatentAttentionSpec(
                hidden_size=W, num_heads=int(mx["heads"]), plain_dim=int(mx["dim"]), rot_dim=int(mx["rot_dim"]),
                value_dim=int(mx["vdim"]), latent_dim=int(mx["kv_rank"]), scale=float(mx["scale"]), position=position,
                latent_norm_eps=eps, prefix="mix", query_latent_dim=int(mx["q_rank"]), window=_mask(mx, where),
                sink="sink")
        return StateSpaceSpec(hidden_size=W, num_heads=int(mx["heads"]), value_dim=int(mx["vdim"]),
                              state_dim=int(mx["state"]), groups=int(mx["groups"]), norm_groups=int(mx["norm_groups"]),
                              conv_taps=int(mx["conv"]), norm_eps=eps, prefix="mix")

    def to_spec(self) -> ModelSpec:
        eps, W = self.norm_eps, self.width
        conv = None if self.conv_taps is None else (self.conv_taps, ("canon1", "canon2"))
        layers, unused = [], []
        for i, layer in enumerate(self.layers):
            ml = layer.get("mlp")
            ff = None if ml is None else DenseMLPSpec(hidden_size=W, intermediate_size=int(ml["ff"]), activation="relu2",
                                                      prefix="mlp")
            layers.append(LayerSpec(prefix=f"l{i}", mixer=self._mixer(layer["type"], layer["mixer"], f"layers[{i}].mixer"),
                                    feed_forward=ff, mixer_norm=NormSpec(W, eps, "norm1", offset=1.0),
                                    ffn_norm=None if ff is None else NormSpec(W, eps, "norm2", offset=1.0),
                                    kind="pre_norm", input_conv=conv))
            if ff is None:          # a folder may hold the second norm and convolution of a layer that has no use for them
                unused += [f"l{i}.norm2", f"l{i}.canon2"]
        spec = ModelSpec(architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=W, layers=tuple(layers),
                         final_norm=NormSpec(W, eps, "final.norm", offset=1.0), embedding_name="embed",
                         lm_head_name="head", logit_scale=self.logit_scale, unused_tensors=tuple(unused))
        spec.validate()
        return spec
