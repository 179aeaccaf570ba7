"""Test material for the Gogivik design: small configurations that differ in every size and option, and a
model-folder writer that is independent of the product's."""

from __future__ import annotations

import json
from pathlib import Path

import torch


def attention(heads, kv, dim, vdim, chunk, rot_dims=None, base=10000.0, factor=None, scale=None):
    rot = {"base": base, "dims": rot_dims if rot_dims is not None else dim}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": chunk}, "rot": rot,
                      "scale": scale if scale is not None else dim ** -0.5}}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, base=100000.0, scale=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "mask": {"size": window}, "rot": {"base": base, "dims": rot_dim},
                      "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}}


def mamba(heads, vdim, state, groups, norm_groups, conv):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups,
                                        "norm_groups": norm_groups, "conv": conv}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def layer(mixer: dict, mlp) -> dict:
    return {**mixer, "mlp": mlp}


def config(vocab, width, layers, eps=1e-5, taps=3, logit_scale=None):
    c = {"architecture": "Gogivik", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
         "canon": {"taps": taps}}
    if logit_scale is not None:
        c["logit_scale"] = logit_scale
    return c


# three key/value heads under six query heads, values narrower than keys, a rotation over half of every key head with
# scaled frequencies, chunks that no page size divides; a state-space layer without a feed-forward whose norm covers
# all heads at once; latent attention with values wider than the latent's heads, convolutions of two taps
GA = config(200, 64, [layer(attention(6, 3, 16, 8, chunk=20, rot_dims=8, factor=4.0), dense(48)),
                      layer(mamba(4, 8, 16, groups=2, norm_groups=1, conv=3), None),
                      layer(latent(4, 16, 8, 24, kv_rank=24, q_rank=12, window=17), dense(40))],
            eps=1e-6, taps=2, logit_scale=1.5)
# nothing a multiple of 8: latent rows of 34 elements, one key/value head under three, a norm group that ends in the
# middle of a head, a group of B and C per head, no logit scale, four taps
GB = config(131, 72, [layer(latent(3, 20, 6, 12, kv_rank=28, q_rank=10, window=9), None),
                      layer(attention(3, 1, 20, 12, chunk=7, base=2e4), dense(100)),
                      layer(mamba(3, 8, 5, groups=3, norm_groups=2, conv=2), dense(36))], eps=3e-6, taps=4)
# sizes at which the tensor-core kernels run in bfloat16: keys and values of 64 (the kernel for equal sizes), keys of
# 32 with values of 64 (the kernel per pair of sizes), latent rows of 80, a state of 64 channels
GC = config(320, 128, [layer(attention(8, 2, 64, 64, chunk=48, rot_dims=32, factor=2.0), dense(256)),
                       layer(mamba(8, 16, 64, groups=1, norm_groups=4, conv=4), dense(64)),
                       layer(attention(4, 4, 32, 64, chunk=33, base=5e5), None),
                       layer(latent(8, 32, 16, 32, kv_rank=64, q_rank=48, window=40), dense(128))], taps=3, logit_scale=0.5)
# one head everywhere, convolutions of one tap (a scaling), a chunk longer than any sequence, a window of one position
# (a query sees itself and the sink)
GD = config(90, 40, [layer(attention(1, 1, 16, 16, chunk=1000, rot_dims=4, factor=2.0), dense(8)),
                     layer(latent(1, 8, 2, 6, kv_rank=8, q_rank=4, window=1), None),
                     layer(mamba(1, 6, 4, groups=1, norm_groups=1, conv=1), dense(24))], taps=1, logit_scale=3.0)
# heads of 128 with values of 128, latent rows of 128 (112 + 16), a state of 128 channels with values of 64, five taps
GE = config(150, 96, [layer(attention(4, 2, 128, 128, chunk=64, rot_dims=64), dense(64)),
                      layer(latent(4, 48, 16, 40, kv_rank=112, q_rank=32, window=50), dense(40)),
                      layer(mamba(2, 64, 128, groups=2, norm_groups=2, conv=4), None)], taps=5)
CONFIGS = {"ga": GA, "gb": GB, "gc": GC, "gd": GD, "ge": GE}
PAGE = {"ga": 16, "gb": 8, "gc": 16, "gd": 4, "ge": 32}


def tensor_shapes(c: dict) -> dict:
    W, V = c["width"], c["vocab"]
    taps = c["canon"]["taps"]
    shapes = {"embed": (V, W), "head": (V, W), "final.norm": (W,)}
    for i, ly in enumerate(c["layers"]):
        p, mx = f"l{i}", ly["mixer"]
        shapes.update({f"{p}.norm1": (W,), f"{p}.canon1": (W, taps)})
        if ly["type"] == "attention":
            H, G, D, E = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            shapes.update({f"{p}.mix.q": (H * D, W), f"{p}.mix.k": (G * D, W), f"{p}.mix.v": (G * E, W),
                           f"{p}.mix.q.norm": (D,), f"{p}.mix.k.norm": (D,), f"{p}.mix.o": (W, H * E)})
        elif ly["type"] == "latent_attention":
            H, D, R, E, C, Q = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"], mx["q_rank"]
            shapes.update({f"{p}.mix.dq": (Q, W), f"{p}.mix.dq.norm": (Q,), f"{p}.mix.uq": (H * (D + R), Q),
                           f"{p}.mix.dkv": (C + R, W), f"{p}.mix.dkv.norm": (C,), f"{p}.mix.uk": (H * D, C),
                           f"{p}.mix.uv": (H * E, C), f"{p}.mix.sink": (H,), f"{p}.mix.o": (W, H * E)})
        else:
            H, E, N, G = mx["heads"], mx["vdim"], mx["state"], mx["groups"]
            inner, ch = H * E, H * E + 2 * G * N
            shapes.update({f"{p}.mix.in": (2 * inner + 2 * G * N + H, W), f"{p}.mix.conv": (ch, mx["conv"]),
                           f"{p}.mix.conv.b": (ch,), f"{p}.mix.dt_bias": (H,), f"{p}.mix.A_log": (H,), f"{p}.mix.D": (H,),
                           f"{p}.mix.norm": (inner,), f"{p}.mix.o": (W, inner)})
        if ly["mlp"] is not None:
            shapes.update({f"{p}.norm2": (W,), f"{p}.canon2": (W, taps), f"{p}.mlp.up": (ly["mlp"]["ff"], W),
                           f"{p}.mlp.down": (W, ly["mlp"]["ff"])})
    return shapes


def make_weights(c: dict, seed: int, up_scale: float = 1.5) -> dict:
    """Random float32 weights: matrices N(0, 1.5/sqrt(fan_in)) (the feed-forwards' first matrices `up_scale` instead
    of 1.5: their results are squared), the embedding of order one, the layers' norm weights N(0, 0.1) (one is added to them) (the
    query, key, latent and state-space norms around one), convolutions N(0, 0.5), sinks N(0, 1), A_log around -1, step
    biases around 0, skips around 1."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(c).items():
        z = torch.randn(shape, generator=g, dtype=torch.float32)
        last = name.rsplit(".", 1)[-1]
        if name == "embed":
            out[name] = z
        elif last in ("norm1", "norm2") or name == "final.norm":
            out[name] = 0.1 * z
        elif last in ("canon1", "canon2", "conv"):
            out[name] = 0.5 * z
        elif last == "sink":
            out[name] = z
        elif last == "A_log":
            out[name] = -1.0 + 0.5 * z
        elif last in ("dt_bias", "b"):
            out[name] = 0.3 * z
        elif last == "D":
            out[name] = 1.0 + 0.2 * z
        elif len(shape) == 1:
            out[name] = 1.0 + 0.1 * z
        elif name.endswith(".mlp.up"):
            out[name] = (up_scale / shape[1] ** 0.5) * z
        else:
            out[name] = (1.5 / shape[1] ** 0.5) * z
    return out


def stored(weights: dict) -> dict:
    """The values that the folder holds (bfloat16), as float64: both sides compute from the same numbers."""
    return {k: v.to(torch.bfloat16).to(torch.float64) for k, v in weights.items()}


def write_folder(folder, c: dict, weights: dict, dtype=torch.bfloat16) -> Path:
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(c))
    save_file({k: v.to(dtype).contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return folder
