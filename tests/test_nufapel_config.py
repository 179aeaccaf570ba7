"""Nufapel: config.json -> configuration -> ModelSpec, and the plain implementation's mechanisms, on the CPU."""

from __future__ import annotations

import copy
import math

import pytest
import torch

from jax_vllm_b200 import registry
from jax_vllm_b200.models.nufapel import NufapelConfig
from jax_vllm_b200.parts import BuildContext, Model
from jax_vllm_b200.parts.base import FixedStateNeed, PagedKVNeed
from jax_vllm_b200.parts.general_attention import distance_buckets
from tests.nufapel_util import CONFIGS, config, config_json, delta, dense, layer, moe, pair, tensor_shapes
from tests.plain import nufapel_plain as npl


@pytest.mark.parametrize("tag", sorted(CONFIGS))
def test_tensor_names_shapes_and_round_trip(tag):
    """Every tensor of the folder under its name; the sizes that only tensors carry (rows of the bias table, rank of
    the decay's projection) are open until the weights are bound."""
    c = CONFIGS[tag]
    cfg = registry.config_from_dict(config_json(c))
    assert isinstance(cfg, NufapelConfig)
    assert NufapelConfig.from_dict(cfg.to_dict()) == cfg
    model = Model(cfg.to_spec(), BuildContext(dtype=torch.float32, device=torch.device("cpu")))
    got = {k: tuple(v.shape) for k, v in model.tensor_specs().items()}
    want = tensor_shapes(c)
    assert set(got) == set(want)
    for name, shape in want.items():
        assert len(got[name]) == len(shape) and all(g in (-1, s) for g, s in zip(got[name], shape)), name
    opened = {name for name, shape in got.items() if -1 in shape}
    assert all(name.endswith((".rel", ".w1", ".w2")) for name in opened)


def test_run_order_passes_and_what_each_place_keeps():
    five = [layer(delta(1, 8), dense(8)), layer(pair(2, 1, 8, 8, 1, 8, 8), None), layer(delta(2, 4), None),
            layer(pair(1, 1, 4, 4, 1, 4, 4), dense(8)), layer(delta(1, 8), None)]
    for loop, order, starts in ((None, (0, 1, 2, 3, 4), ()),
                                ((0, 5, 2), (0, 1, 2, 3, 4, 0, 1, 2, 3, 4), ((0, 0), (5, 1))),
                                ((1, 3, 3), (0, 1, 2, 1, 2, 1, 2, 3, 4), ((1, 0), (3, 1), (5, 2))),
                                ((4, 5, 1), (0, 1, 2, 3, 4), ((4, 0),))):
        c = config(50, 16, copy.deepcopy(five), loop=loop)
        cfg = registry.config_from_dict(config_json(c))
        assert cfg.run_order() == (order, starts)
        spec = cfg.to_spec()
        assert tuple(spec.run_order()) == order
        assert (spec.pass_vectors is None) == (loop is None)
        plain = npl.run_order(c)
        assert tuple(i for i, _ in plain) == order
        assert tuple((k, t) for k, (_, t) in enumerate(plain) if t is not None) == starts
        # every place of the order keeps a state row of its own; a pair keeps pages and a state row
        needs = Model(spec, BuildContext(dtype=torch.float32, device=torch.device("cpu"))).cache_needs()
        assert len(needs) == len(order)
        for place, need in zip(order, needs):
            if five[place]["type"] == "parallel":
                assert isinstance(need, tuple) and isinstance(need[0], PagedKVNeed) and isinstance(need[1], FixedStateNeed)
            else:
                assert isinstance(need, FixedStateNeed)


def test_what_the_design_does_not_have_is_refused():
    good = config_json(CONFIGS["na"])
    registry.config_from_dict(good)

    def broken(change):
        c = copy.deepcopy(good)
        change(c)
        with pytest.raises((KeyError, ValueError)):
            registry.config_from_dict(c)
    broken(lambda c: c["layers"][0].update(type="window"))
    broken(lambda c: c["layers"][0]["mixer"]["left"].pop("bias_max"))
    broken(lambda c: c["layers"][0]["mixer"]["left"].update(heads=5))              # not a multiple of the key heads
    broken(lambda c: c["layers"][0]["mixer"]["right"].update(gate_cap=0.0))
    broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=5))               # more than the kept groups hold
    broken(lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4))   # 6 experts in 4 groups
    broken(lambda c: c["layers"][1]["mlp"].update(kind="gated"))
    broken(lambda c: c["loop"].update(stop=9))
    broken(lambda c: c.pop("norm"))


def test_a_folder_may_hold_the_second_norm_of_a_layer_without_a_feed_forward():
    from jax_vllm_b200.weights import loader
    c = CONFIGS["nb"]                                     # its first layer has no feed-forward, and it has no loop
    model = Model(registry.config_from_dict(config_json(c)).to_spec(), BuildContext(dtype=torch.float32, device=torch.device("cpu")))
    index = {name: (None, [16 if d == -1 else d for d in spec.shape], "BF16") for name, spec in model.tensor_specs().items()}
    W = c["width"]
    index.update({"l0.norm2": (None, [W], "BF16"), "l0.rg2": (None, [W, W], "BF16"), "loop.step": (None, [1, W], "BF16")})
    loader.check("folder", index, model.tensor_specs(), model.optional_tensors())
    index["l1.rg3"] = (None, [W, W], "BF16")
    with pytest.raises(loader.WeightError) as err:
        loader.check("folder", index, model.tensor_specs(), model.optional_tensors())
    assert err.value.unexpected == ["l1.rg3"]


def test_distance_buckets_of_the_product_and_of_the_plain_implementation():
    for B, far in ((8, 30), (16, 120), (4, 5), (32, 1024), (6, 17), (12, 100)):
        table = distance_buckets(B, far)
        assert table == [npl.distance_bucket(n, B, far) for n in range(far + 1)]
        assert table[:B // 2] == list(range(B // 2)) and table[-1] == B - 1 and max(table) == B - 1
        assert all(b1 >= b0 for b0, b1 in zip(table, table[1:]))
        assert npl.distance_bucket(far + 1000, B, far) == B - 1


def test_plain_implementation_mechanisms():
    """Identities that hold whatever the weights: the delta rule without decay and removal is a sum of outer products;
    the memory scanned in two halves carries on from its state; the sink with a very negative value leaves an
    ordinary softmax; groups that keep everything choose the plain top experts."""
    g = torch.Generator().manual_seed(1)
    T, H, D, V = 9, 2, 5, 3
    r, k, v = (torch.randn(T, H, n, generator=g, dtype=torch.float64) for n in (D, D, V))
    ones, zeros = torch.ones(T, H, D, dtype=torch.float64), torch.zeros(T, H, D, dtype=torch.float64)
    o, S = npl.delta_scan(r, k, v, ones, zeros)
    assert torch.allclose(S, torch.einsum("thk,thv->hkv", k, v))
    assert torch.allclose(o[-1], torch.einsum("hkv,hk->hv", S, r[-1]))
    gi, gf = npl.capped_gates(torch.randn(T, H, generator=g, dtype=torch.float64) * 5, torch.randn(T, H, generator=g, dtype=torch.float64) * 5, 4.0)
    assert gi.abs().max() <= 4.0 and gf.max() < 0 and gf.min() >= math.log(1 / (1 + math.exp(4.0))) - 1e-12
    whole, end = npl.memory_scan(r, k, v, gi, gf)
    first, mid = npl.memory_scan(r[:4], k[:4], v[:4], gi[:4], gf[:4])
    second, end2 = npl.memory_scan(r[4:], k[4:], v[4:], gi[4:], gf[4:], mid)
    assert torch.allclose(torch.cat([first, second]), whole) and all(torch.allclose(a, b) for a, b in zip(end, end2))
    q = torch.randn(T, H, D, generator=g, dtype=torch.float64)
    rel = torch.zeros(4, H, dtype=torch.float64)
    temp = torch.ones(H, dtype=torch.float64)
    plain = npl.biased_sink_attend(q, k, v, 0.3, temp, rel, 9, torch.full((H,), -1e9, dtype=torch.float64))
    s = torch.einsum("ihd,jhd->hij", q, k) * 0.3
    s = s.masked_fill(torch.arange(T)[None, :] > torch.arange(T)[:, None], -math.inf)
    assert torch.allclose(plain, torch.einsum("hij,jhv->ihv", torch.softmax(s, -1), v))
    heavy = npl.biased_sink_attend(q, k, v, 0.3, temp, rel, 9, torch.full((H,), 50.0, dtype=torch.float64))
    assert heavy.abs().max() < 1e-12                     # a sink that outweighs every key leaves nothing
    z = torch.randn(20, 8, generator=g, dtype=torch.float64)
    idx, w = npl.route(z, 3, 4, 4, 2.0)
    assert torch.equal(idx, torch.sigmoid(z).topk(3, dim=-1).indices)
    assert torch.allclose(w.sum(-1), torch.full((20,), 2.0, dtype=torch.float64))
    idx, _ = npl.route(z, 2, 4, 1, 1.0)
    assert bool((idx // 2 == (idx // 2)[:, :1]).all())    # one group kept: both chosen experts are neighbours
