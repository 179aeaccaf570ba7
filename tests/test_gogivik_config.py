"""Gogivik: config.json -> configuration -> ModelSpec, and the plain implementation's mechanisms, on the CPU."""

from __future__ import annotations

import copy

import pytest
import torch

from jax_vllm_b200 import registry
from jax_vllm_b200.cache import CacheManager
from jax_vllm_b200.models.gogivik import GogivikConfig
from jax_vllm_b200.parts import BuildContext, Model
from jax_vllm_b200.parts.base import FixedStateNeed, PagedKVNeed
from tests.gogivik_util import CONFIGS, attention, config, dense, latent, layer, make_weights, mamba, stored, tensor_shapes
from tests.plain import gogivik_plain as gp


def cpu_model(c):
    cfg = registry.config_from_dict(c)
    return cfg, Model(cfg.to_spec(), BuildContext(dtype=torch.float32, device=torch.device("cpu")))


@pytest.mark.parametrize("tag", sorted(CONFIGS))
def test_tensor_names_shapes_and_round_trip(tag):
    c = CONFIGS[tag]
    cfg, model = cpu_model(c)
    assert isinstance(cfg, GogivikConfig)
    assert GogivikConfig.from_dict(cfg.to_dict()) == cfg
    assert {k: tuple(v.shape) for k, v in model.tensor_specs().items()} == tensor_shapes(c)


def test_what_every_layer_keeps():
    """Pages for the attention layers (chunked ones give pages back by chunk, latent ones by window and keep one row a
    token), one state row for a state-space layer, and behind each a row of taps - 1 inputs per sublayer."""
    c = CONFIGS["ga"]
    _, model = cpu_model(c)
    needs = model.cache_needs()
    W, taps = c["width"], c["canon"]["taps"]
    att, ssm, lat = needs
    assert att[0] == PagedKVNeed(3, 16, None, v_heads=3, v_head_dim=8, chunk=20) and len(att) == 3
    assert lat[0] == PagedKVNeed(1, 32, 17, shared_kv=True) and len(lat) == 3
    assert ssm[0] == FixedStateNeed((4 * 16 * 8 + 2 * (4 * 8 + 2 * 2 * 16),), torch.float32) and len(ssm) == 2   # no feed-forward
    assert all(n == FixedStateNeed(((taps - 1) * W,), torch.float32) for need in needs for n in need[1:])
    # one tap: the convolution keeps nothing
    _, model = cpu_model(CONFIGS["gd"])
    assert all(not isinstance(need, tuple) for need in model.cache_needs())


def test_pages_of_a_chunk_that_is_over_go_back():
    """A chunked layer's pages are given back once the next query's chunk starts behind them."""
    need = PagedKVNeed(2, 16, None, chunk=20)
    cm = CacheManager([need], page_size=8, num_pages=16, max_live=2, prefix_cache=False)
    rc = cm.admit("a")
    cm.grow(rc, 19)
    cm.commit(rc, list(range(19)))
    assert rc.freed_upto == [0]                      # position 19 is still in the first chunk
    cm.grow(rc, 41)
    cm.commit(rc, list(range(22)))                   # 41 tokens: the next query is in chunk [40, 60)
    assert rc.freed_upto == [5] and list(rc.tables[0])[:5] == [-1] * 5 and rc.tables[0][5] >= 0
    cm.check()
    cm.release("a")
    assert cm.groups[0].pool.num_free == 16


def test_refusals():
    base = CONFIGS["ga"]

    def changed(f):
        c = copy.deepcopy(base)
        f(c)
        return c

    for bad in (changed(lambda c: c["layers"][0].__setitem__("type", "unknown")),
                changed(lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 4)),
                changed(lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7)),
                changed(lambda c: c["layers"][2]["mixer"]["rot"].__setitem__("dims", 4)),
                changed(lambda c: c["layers"][1]["mixer"].__setitem__("groups", 3)),
                changed(lambda c: c["layers"][1]["mixer"].__setitem__("norm_groups", 5)),
                changed(lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe")),
                changed(lambda c: c["canon"].__setitem__("taps", 0)),
                changed(lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0))):
        with pytest.raises((ValueError, KeyError)):
            registry.config_from_dict(bad)
    with pytest.raises(KeyError):
        registry.config_from_dict({k: v for k, v in base.items() if k != "norm"})


# ------------------------------------------------------------ the plain implementation's own identities
def test_plain_tap_conv_and_rotation():
    g = torch.Generator().manual_seed(1)
    u = torch.randn((9, 5), generator=g, dtype=torch.float64)
    w = torch.randn((5, 3), generator=g, dtype=torch.float64)
    out = gp.tap_conv(u, w)
    assert torch.allclose(out[0], w[:, 2] * u[0]) and torch.allclose(out[4], w[:, 0] * u[2] + w[:, 1] * u[3] + w[:, 2] * u[4])
    f = gp.frequencies(100.0, 6)
    y = torch.randn((4, 2, 10), generator=g, dtype=torch.float64)
    pos = torch.tensor([0, 3, 7, 50])
    for layout in ("halves", "interleaved"):
        r = gp.rotate(y, pos, f, layout)
        assert torch.allclose(r[0], y[0]) and torch.allclose(r[..., 6:], y[..., 6:])          # position 0, and what is not rotated
        assert torch.allclose(gp.rotate(r, pos, f, layout, sign=-1.0), y)
        assert torch.allclose((r * r).sum(-1), (y * y).sum(-1))
    # rotated keys and queries: the score depends on the distance only
    a, b = torch.randn((1, 1, 6), generator=g, dtype=torch.float64), torch.randn((1, 1, 6), generator=g, dtype=torch.float64)
    s = [float((gp.rotate(a, torch.tensor([p + 4]), f, "halves") * gp.rotate(b, torch.tensor([p]), f, "halves")).sum()) for p in (0, 9)]
    assert abs(s[0] - s[1]) < 1e-12


def test_plain_masks_and_sink():
    m = gp.visible(10, window=3)
    assert m[5].tolist() == [False] * 3 + [True] * 3 + [False] * 4
    m = gp.visible(10, chunk=4)
    assert m[5].tolist() == [False] * 4 + [True] * 2 + [False] * 4 and m[4].tolist() == [False] * 4 + [True] + [False] * 5
    g = torch.Generator().manual_seed(2)
    q, k, v = (torch.randn((6, 2, 4), generator=g, dtype=torch.float64) for _ in range(3))
    full = gp.visible(6)
    plain = gp.softmax_attend(q, k, v, 0.5, full)
    gone = gp.softmax_attend(q, k, v, 0.5, full, sink=torch.full((2,), -80.0, dtype=torch.float64))
    heavy = gp.softmax_attend(q, k, v, 0.5, full, sink=torch.full((2,), 80.0, dtype=torch.float64))
    assert torch.allclose(plain, gone) and heavy.abs().max() < 1e-20


def test_plain_state_space_is_a_decayed_sum():
    """One head, one state channel, no convolution: y_t = sum_s prod_(s < r <= t) a_r dt_s B_s C_t x_s + D x_t."""
    c = config(20, 8, [layer(mamba(1, 2, 1, 1, 1, conv=1), None)], taps=1)
    w = stored(make_weights(c, 3))
    g = torch.Generator().manual_seed(4)
    u = torch.randn((5, 8), generator=g, dtype=torch.float64)
    mx = c["layers"][0]["mixer"]
    got = gp.mamba2(u, w, "l0.mix", mx, 1e-5)
    row = u @ w["l0.mix.in"].T
    z, xbc, dt = row[:, :2], row[:, 2:6], row[:, 6:]
    xbc = torch.nn.functional.silu(xbc * w["l0.mix.conv"][:, 0] + w["l0.mix.conv.b"])
    x, B, C = xbc[:, :2], xbc[:, 2], xbc[:, 3]
    dt = torch.nn.functional.softplus(dt[:, 0] + w["l0.mix.dt_bias"][0])
    a = torch.exp(-torch.exp(w["l0.mix.A_log"][0]) * dt)
    y = torch.zeros((5, 2), dtype=torch.float64)
    for t in range(5):
        for s in range(t + 1):
            y[t] += a[s + 1:t + 1].prod() * dt[s] * B[s] * C[t] * x[s]
        y[t] += w["l0.mix.D"][0] * x[t]
    y = gp.unit(y * torch.nn.functional.silu(z), 1e-5) * w["l0.mix.norm"]
    assert torch.allclose(got, y @ w["l0.mix.o"].T, atol=1e-12)
