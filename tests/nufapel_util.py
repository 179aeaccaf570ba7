"""Test material for the Nufapel design: small configurations that differ in every size and option, and a
model-folder writer that is independent of the product's."""

from __future__ import annotations

import json
from pathlib import Path

import torch


def pair(heads, kv, dim, vdim, mem_heads, mem_dim, mem_vdim, scale=None, bias_max=40, buckets=8, cap=15.0):
    """A layer of two mixers side by side: attention (left) and a matrix memory (right)."""
    return {"type": "parallel", "buckets": buckets,
            "mixer": {"left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "bias_max": bias_max,
                               "scale": scale if scale is not None else dim ** -0.5},
                      "right": {"heads": mem_heads, "dim": mem_dim, "vdim": mem_vdim, "gate_cap": cap}}}


def delta(heads, dim, rank=8):
    return {"type": "general_delta", "rank": rank, "mixer": {"heads": heads, "dim": dim}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, groups, keep, ff, scale=1.5, limit=2.0):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}, "scale": scale}}


def layer(mixer: dict, mlp) -> dict:
    """`buckets` and `rank` are sizes that only tensors carry: they are kept beside the layer for `tensor_shapes`
    and do not enter config.json."""
    return {**mixer, "mlp": mlp}


def config(vocab, width, layers, eps=1e-5, loop=None, softcap=30.0, max_positions=512):
    c = {"architecture": "Nufapel", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
         "max_positions": max_positions, "logit_softcap": softcap}
    if loop is not None:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


def config_json(c: dict) -> dict:
    """What goes into config.json: the layers without the sizes that only tensors carry."""
    out = dict(c)
    out["layers"] = [{k: v for k, v in ly.items() if k not in ("buckets", "rank")} for ly in c["layers"]]
    return out


# three key/value heads under six query heads, values narrower than keys, a memory with values wider than keys, routed
# experts in three groups of which two are kept (top 3), a loop over the last two layers that runs twice
NA = config(200, 64, [layer(pair(6, 3, 16, 8, 2, 8, 24, bias_max=30, buckets=8), dense(48)),
                      layer(delta(2, 16, rank=4), moe(6, 3, 3, 2, 24, scale=1.5, limit=2.0)),
                      layer(pair(2, 2, 24, 40, 3, 20, 12, bias_max=100, buckets=12, cap=8.0), moe(4, 1, 1, 1, 16, scale=0.7, limit=1.0))],
            eps=1e-6, loop=(1, 3, 2), softcap=20.0)
# nothing a multiple of 8, heads of one kind only in a layer, a layer without a feed-forward, no loop, one expert a group
NB = config(131, 72, [layer(delta(3, 20, rank=5), None),
                      layer(pair(3, 1, 20, 12, 1, 36, 28, bias_max=17, buckets=6), moe(5, 2, 5, 3, 20, scale=2.0, limit=3.0)),
                      layer(delta(1, 40, rank=16), dense(100))], eps=3e-6, softcap=50.0)
# sizes at which tensor-core products and wider scans run: keys of 128 and 64, a loop from the first layer that runs
# three times before the last layer
NC = config(320, 128, [layer(pair(8, 2, 64, 64, 2, 128, 64, bias_max=200, buckets=32), moe(8, 2, 4, 2, 128, limit=2.0)),
                       layer(delta(2, 128, rank=32), dense(256)),
                       layer(pair(4, 4, 32, 32, 4, 32, 32, bias_max=64, buckets=16), None)], eps=1e-5, loop=(0, 2, 3))
# one layer, one head everywhere, a loop of one pass
ND = config(90, 40, [layer(pair(1, 1, 16, 24, 1, 12, 6, bias_max=9, buckets=4), dense(8))], eps=1e-5, loop=(0, 1, 1))
# attention heads of 128 with values of 128 (prompt tiles of 64 tokens on the tcgen05 kernel in bfloat16), a memory with
# keys of 256, a delta rule with heads of 200 (not a multiple of 16), a table with an odd number of heads' columns
NE = config(150, 96, [layer(pair(4, 2, 128, 128, 1, 256, 16, bias_max=50, buckets=10), dense(64)),
                      layer(delta(1, 200, rank=3), None),
                      layer(pair(3, 3, 128, 128, 2, 16, 48, bias_max=300, buckets=20, cap=10.0), dense(40))],
            eps=1e-5, loop=(0, 1, 2), softcap=25.0)
CONFIGS = {"na": NA, "nb": NB, "nc": NC, "nd": ND, "ne": NE}
PAGE = {"na": 16, "nb": 8, "nc": 16, "nd": 4, "ne": 32}


def tensor_shapes(c: dict) -> dict:
    W, V = c["width"], c["vocab"]
    shapes = {"embed": (V, W), "pos": (c["max_positions"], W), "head": (V, W)}
    for name in ("final.norm",):
        shapes.update({name: (W,), f"{name}.b": (W,), f"{name}.alpha": ()})
    if "loop" in c:
        shapes["loop.step"] = (c["loop"]["times"], W)
    for i, ly in enumerate(c["layers"]):
        p, mx = f"l{i}", ly["mixer"]
        subs = ("1", "2") if ly["mlp"] is not None else ("1",)
        for s in subs:
            shapes.update({f"{p}.norm{s}": (W,), f"{p}.norm{s}.b": (W,), f"{p}.norm{s}.alpha": (),
                           f"{p}.rg{s}": (W, W), f"{p}.rg{s}.b": (W,)})
        if ly["type"] == "general_delta":
            HD, R = mx["heads"] * mx["dim"], ly["rank"]
            shapes.update({f"{p}.mix.{n}": (HD, W) for n in ("r", "k", "v", "g", "a")})
            shapes.update({f"{p}.mix.a.b": (HD,), f"{p}.mix.w1": (R, W), f"{p}.mix.w2": (HD, R), f"{p}.mix.w0": (HD,),
                           f"{p}.mix.norm": (HD,), f"{p}.mix.o": (W, HD)})
        else:
            le, ri = mx["left"], mx["right"]
            H, G, D, E = le["heads"], le["kv_heads"], le["dim"], le["vdim"]
            shapes.update({f"{p}.mix.left.q": (H * D, W), f"{p}.mix.left.k": (G * D, W), f"{p}.mix.left.v": (G * E, W),
                           f"{p}.mix.left.rel": (ly["buckets"], H), f"{p}.mix.left.temp": (H,), f"{p}.mix.left.sink": (H,),
                           f"{p}.mix.left.g": (H, W), f"{p}.mix.left.o": (W, H * E)})
            H, D, E = ri["heads"], ri["dim"], ri["vdim"]
            shapes.update({f"{p}.mix.right.q": (H * D, W), f"{p}.mix.right.k": (H * D, W), f"{p}.mix.right.v": (H * E, W),
                           f"{p}.mix.right.g": (H * E, W), f"{p}.mix.right.o": (W, H * E), f"{p}.mix.right.norm": (H * E,),
                           f"{p}.mix.right.i": (H, W), f"{p}.mix.right.i.b": (H,), f"{p}.mix.right.f": (H, W),
                           f"{p}.mix.right.f.b": (H,), f"{p}.mix.left.out": (W,), f"{p}.mix.right.out": (W,)})
        ml = ly["mlp"]
        if ml is None:
            continue
        if ml["kind"] == "dense":
            shapes.update({f"{p}.mlp.up": (ml["ff"], W), f"{p}.mlp.down": (W, ml["ff"])})
        else:
            F = ml["expert"]["ff"]
            shapes[f"{p}.mlp.router"] = (ml["router"]["experts"], W)
            for e in range(ml["router"]["experts"]):
                shapes.update({f"{p}.mlp.e{e}.gate": (F, W), f"{p}.mlp.e{e}.up": (F, W), f"{p}.mlp.e{e}.down": (W, F)})
    return shapes


def make_weights(c: dict, seed: int) -> dict:
    """Random float32 weights: matrices N(0, 1.5/sqrt(fan_in)), embedding and positions of order one, norm weights
    1 + N(0, 0.1), norm slopes near 0.7, biases N(0, 0.3), distance biases and sinks N(0, 1), temperatures around 1.
    Router matrices are larger, so that the scores are spread and no choice is a close call."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(c).items():
        z = torch.randn(shape, generator=g, dtype=torch.float32)
        last = name.rsplit(".", 1)[-1]
        if last == "alpha":
            out[name] = 0.7 + 0.1 * z
        elif name in ("embed",):
            out[name] = z
        elif name in ("pos", "loop.step"):
            out[name] = 0.5 * z
        elif last in ("rel", "sink"):
            out[name] = z
        elif last == "temp":
            out[name] = 1.0 + 0.2 * z
        elif last == "router":
            out[name] = (4.0 / shape[1] ** 0.5) * z
        elif last in ("b", "w0"):
            out[name] = 0.3 * z
        elif len(shape) == 1:
            out[name] = 1.0 + 0.1 * z
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
    (folder / "config.json").write_text(json.dumps(config_json(c)))
    save_file({k: v.to(dtype).contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return folder
