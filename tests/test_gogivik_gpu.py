"""The Gogivik design in the engine against the plain implementation (tests/plain/gogivik_plain.py): every mechanism
alone, then models of several sizes through the replay program's class (whole, last tokens one by one, portions down
to two tokens, unequal requests side by side in reused pages and state slots), special weights where random ones would
hide a fault, and greedy generation through the entry point and its scheduler."""

from __future__ import annotations

import copy
import json
import math
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from tests.gogivik_util import (CONFIGS, PAGE, attention, config, dense, latent, layer, make_weights, mamba, stored,
                                write_folder)
from tests.plain import gogivik_plain as gp
from tests.test_nufapel_gpu import mixed_trace, scrambled_pages
from tests.test_replay_gpu import limits
from tests.util import collect, portions, prefix_then_single, random_tokens, whole

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
LENGTHS = {"ga": [70, 45, 100, 33, 52], "gb": [90, 38, 64, 51, 27], "gc": [200, 70, 150, 40, 66], "gd": [61, 40, 83, 35, 20],
           "ge": [170, 60, 100, 37, 45]}


def oracle(c, w, tokens):
    return gp.forward(c, w, tokens).to(torch.float32)


def rounding_error(c, w, tokens):
    """Per position, how far the plain logits move when the operands and the result of every matrix product are
    rounded to bfloat16 and nothing else is: what rounding alone does to this model at this token."""
    bf = lambda x: x.to(torch.bfloat16).to(torch.float64)
    exact = gp.forward(c, w, tokens)
    plain_matmul = torch.Tensor.__matmul__
    torch.Tensor.__matmul__ = lambda a, b: bf(plain_matmul(bf(a), bf(b)))
    try:
        rounded = gp.forward(c, w, tokens)
    finally:
        torch.Tensor.__matmul__ = plain_matmul
    return (rounded - exact).abs().max(dim=1).values


def compare(steps, out_dir, vocab, want, dtype, case=None, rounding=None):
    """Every written row against the oracle's.  32-bit holds every position and the greedy token.  In bfloat16 one
    position in fifty (or one) may be over the limit by up to half of it.  `rounding` (request -> `rounding_error`):
    a bfloat16 position's limit is at least three times what rounding alone does there, for models drawn at random
    whose narrow heads let two terms cancel before a unit norm at some tokens."""
    from tests.conftest import record_worst
    got = collect(steps, out_dir, vocab)
    worst, lim_of_worst, total, slightly = 0.0, 0.0, 0, 0
    for rid, rows in got.items():
        lim_all = limits(dtype, want[rid])
        for pos, row in rows.items():
            total += 1
            lim = lim_all
            if rounding is not None and dtype != "float32":
                lim = max(lim, 3.0 * float(rounding[rid][pos]))
            w = want[rid][pos]
            diff = (torch.from_numpy(row.copy()) - w).abs().max().item()
            assert math.isfinite(diff), f"{rid} position {pos}: not a number"
            if dtype != "float32" and lim < diff <= 1.5 * lim:
                slightly += 1
                continue
            assert diff <= lim, f"{rid} position {pos}: |diff| {diff:.3e} > {lim:.3e}"
            if diff >= worst:
                worst, lim_of_worst = diff, lim
            if dtype == "float32":
                top2 = w.topk(2).values
                assert int(row.argmax()) == int(w.argmax()) or float(top2[0] - top2[1]) < 1e-4
    # the rounding of a run is one draw of what `rounding_error` estimates: with it, one position in ten may be over
    share = 0.1 if rounding is not None else 0.02
    assert slightly <= max(1, share * total), f"{slightly} of {total} positions are over the limit"
    if case is not None:
        record_worst(case, dtype, worst, lim_of_worst)
    return got


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def setup(request, tmp_path_factory):
    tag = request.param
    c = CONFIGS[tag]
    weights = make_weights(c, seed=5)
    folder = write_folder(tmp_path_factory.mktemp(f"gogivik_{tag}"), c, weights)
    w = stored(weights)
    seqs = {f"r{i}": random_tokens(n, c["vocab"], seed=20 + i) for i, n in enumerate(LENGTHS[tag])}
    want = {rid: oracle(c, w, t) for rid, t in seqs.items()}
    assert all(v.abs().max() > 1.0 for v in want.values())     # logits of order one, not a flat model
    return tag, folder, seqs, want


def replay(folder, tag, dtype, steps, out_dir, max_tokens, **switches):
    from jax_vllm_b200.engine.replay import Replayer
    rep = Replayer(folder, dtype, out_dir, max_tokens=max_tokens, page_size=PAGE[tag], **switches)
    rep.run_stream(json.dumps(s) for s in steps)
    rep.cache.check()
    assert not rep.cache.live
    return rep


def entries_of(lengths, slots):
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32).cuda()
    return cu, torch.tensor(slots, dtype=torch.int32).cuda()


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("mode", ["residual", "bias_silu"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,C", [(1, 40), (2, 33), (3, 64), (4, 200), (5, 7), (8, 130)])
def test_short_convolution_alone(taps, C, dtype, mode):
    """Four entries of unequal length (one longer than two segments, one of a single token, one shorter than the
    state) whose histories lie in slots given out of order; a second call carries on from what the first left; an
    unused slot stays as it was.  The input is a column range of wider rows."""
    from jax_vllm_b200 import ops
    g = torch.Generator().manual_seed(taps * 100 + C)
    K = taps - 1
    first, second, slots, n_slots = [150, 1, 2, 9], [1, 3, 66, 1], [3, 0, 4, 1], 6
    w = (0.5 * torch.randn((C, taps), generator=g)).to(dtype)
    b = (0.3 * torch.randn(C, generator=g)).to(dtype)
    history = [torch.randn((K, C), generator=g) for _ in first]
    full = [torch.cat([history[e], torch.randn((first[e] + second[e], C), generator=g).to(dtype).float()]) for e in range(4)]
    state = torch.full((n_slots, K * C + 3), 7.0)
    for e, s in enumerate(slots):
        state[s, :K * C] = history[e].reshape(-1)
    state = state.cuda()
    view = state[:, :K * C] if K else None
    done = [0] * 4
    for lengths in (first, second):
        rows = torch.cat([full[e][K + done[e]:K + done[e] + n] for e, n in enumerate(lengths)])
        wide = torch.cat([torch.full((rows.shape[0], 5), float("nan")), rows, torch.full((rows.shape[0], 2), float("nan"))], 1).to(dtype).cuda()
        cu, sl = entries_of(lengths, slots)
        kw = dict(residual=True) if mode == "residual" else dict(bias=b.cuda(), act="silu")
        out = ops.short_conv(wide[:, 5:5 + C], w.cuda(), view, cu, sl, 4, dtype, **kw).float().cpu()
        ops.check_status()
        at = 0
        for e, n in enumerate(lengths):
            seq = full[e][:K + done[e] + n].double()
            conv = gp.tap_conv(seq, w.double(), None if mode == "residual" else b.double())
            want = (seq + conv if mode == "residual" else torch.nn.functional.silu(conv))[K + done[e]:]
            tol = 1e-5 if dtype == torch.float32 else 1.5e-2
            assert (out[at:at + n].double() - want).abs().max() < tol * max(1.0, want.abs().max().item()), (e, lengths)
            at += n
            done[e] += n
            if K:
                assert torch.equal(state[slots[e], :K * C].cpu().view(K, C), full[e][done[e]:done[e] + K]), (e, lengths)
    assert bool((state[2] == 7.0).all() and (state[5] == 7.0).all() and (state[:, K * C:] == 7.0).all())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout", ["halves", "interleaved"])
@pytest.mark.parametrize("Hq,Hk,D,E,rot,normed", [(6, 3, 16, 8, 8, True), (3, 1, 20, 12, 20, True), (4, 4, 32, 64, 2, False),
                                                  (1, 1, 70, 34, 40, True), (8, 2, 128, 128, 64, True)])
def test_heads_prepared_one_by_one(Hq, Hk, D, E, rot, normed, layout, dtype):
    """Norm per head with one shared weight, rotation of a leading part in both layouts with scaled frequencies, values
    unit-normed and rotated by their own position into scrambled pages; the heads' rotation back undoes the values'."""
    from jax_vllm_b200 import ops
    g = torch.Generator().manual_seed(Hq * D + E)
    P, n_pages, eps = 8, 40, 1e-5
    ctx_new = [(37, 21), (0, 3), (130, 1)]
    table = scrambled_pages(ctx_new, P, n_pages, g)
    n = sum(q for _, q in ctx_new)
    pos = torch.cat([torch.arange(c, c + q) for c, q in ctx_new])
    ent = torch.cat([torch.full((q,), e) for e, (_, q) in enumerate(ctx_new)])
    cols = Hq * D + Hk * D + Hk * E
    proj = (1.5 * torch.randn((n, cols + 3), generator=g)).to(dtype)
    qw = (1.0 + 0.2 * torch.randn(D, generator=g)).to(dtype)
    kw = (1.0 + 0.2 * torch.randn(D, generator=g)).to(dtype)
    freq = gp.frequencies(5e4, rot, 4.0).float()
    vfreq = gp.frequencies(5e4, E, 1.0).float()
    kc = torch.zeros((n_pages, P, Hk, D), dtype=dtype).cuda()
    vc = torch.zeros((n_pages, P, Hk, E), dtype=dtype).cuda()
    q_out = torch.empty((n, Hq * D), dtype=dtype).cuda()
    ops.head_prepare(proj.cuda(), 3, 3 + Hq * D, 3 + Hq * D + Hk * D, q_out, pos.int().cuda(), ent.int().cuda(), table.cuda(),
                     freq.cuda(), layout == "interleaved", qw.cuda() if normed else None, kw.cuda() if normed else None, eps,
                     True, vfreq.cuda(), kc, vc, Hq, Hk, Hk, D, E)
    ops.check_status()
    x = proj.double()
    q = x[:, 3:3 + Hq * D].view(n, Hq, D)
    k = x[:, 3 + Hq * D:3 + Hq * D + Hk * D].view(n, Hk, D)
    v = x[:, 3 + Hq * D + Hk * D:3 + cols].view(n, Hk, E)
    if normed:
        q, k = gp.unit(q, eps) * qw.double(), gp.unit(k, eps) * kw.double()
    q, k = gp.rotate(q, pos, freq.double(), layout), gp.rotate(k, pos, freq.double(), layout)
    v = gp.rotate(gp.unit(v, eps), pos, vfreq.double(), layout)
    tol = 2e-5 if dtype == torch.float32 else 1.2e-2
    close = lambda a, b: (a.double().cpu() - b).abs().max().item() < tol * max(1.0, b.abs().max().item())
    assert close(q_out.view(n, Hq, D), q)
    for t in range(n):
        page, slot = int(table[ent[t], pos[t] // P]), int(pos[t] % P)
        assert close(kc[page, slot], k[t]) and close(vc[page, slot], v[t]), t
    # the rotation back, on rows that are a column range, into another type
    wide = torch.zeros((n, Hk * E + 4), dtype=dtype).cuda()
    wide[:, 4:] = torch.stack([vc[int(table[ent[t], pos[t] // P]), int(pos[t] % P)] for t in range(n)]).view(n, Hk * E)
    back = torch.empty((n, Hk * E), dtype=torch.float32).cuda()
    ops.head_rotate(wide[:, 4:], pos.int().cuda(), vfreq.cuda(), layout == "interleaved", Hk, E, sign=-1.0, out=back)
    assert close(back.view(n, Hk, E), gp.unit(x[:, 3 + Hq * D + Hk * D:3 + cols].view(n, Hk, E), eps))


MASK_CASES = {
    # name: (kernel, query heads, key heads, key size, value size)
    "simt32": ("simt", 6, 3, 20, 12), "simt16": ("simt", 3, 1, 40, 40), "sizes_16": ("general", 4, 2, 32, 64),
    "sizes_16_of_128": ("general", 4, 1, 128, 128), "equal_64": ("equal", 8, 2, 64, 64), "equal_128": ("equal", 4, 4, 128, 128),
    "latent_80": ("latent", 8, 1, 80, 64), "latent_144": ("latent", 5, 1, 144, 128), "latent_simt": ("latent_simt", 3, 1, 34, 28),
}


@pytest.mark.parametrize("mask", [("window", 1), ("window", 13), ("window", 64), ("chunk", 7), ("chunk", 48), ("chunk", 1000)])
@pytest.mark.parametrize("name", sorted(MASK_CASES))
def test_windows_chunks_and_sinks_on_every_attention_kernel(name, mask):
    """A prompt portion over several tiles behind earlier context, a short prompt from position 0, and a single token
    whose keys are split into ranges: under a window or chunks, with a sink where the kernel has one.  Scores are
    spread (a sharp softmax), and the plain result with one more visible position differs by far more than the limit."""
    from jax_vllm_b200 import ops
    kernel, Hq, Hk, D, E = MASK_CASES[name]
    dtype = torch.float32 if name == "simt32" else torch.bfloat16
    latent_rows = kernel.startswith("latent")
    sink_on = latent_rows or kernel == "simt" or kernel == "general"
    g = torch.Generator().manual_seed(Hq * D + E + mask[1])
    P, n_pages, scale = 8, 64, 1.3 * D ** -0.5
    ctx_new = [(37, 45), (0, 3), (130, 1)]
    table = scrambled_pages(ctx_new, P, n_pages, g)
    kc = torch.full((n_pages, P, Hk, D), float("nan"), dtype=dtype)
    vc = kc if latent_rows else torch.full((n_pages, P, Hk, E), float("nan"), dtype=dtype)
    window = mask[1] if mask[0] == "window" else None
    chunk = mask[1] if mask[0] == "chunk" else None
    code = ops.mask_code(window, chunk)
    ks, vs, qs = [], [], []
    for e, (c, q) in enumerate(ctx_new):
        k = (torch.randn((c + q, Hk, D), generator=g) * 1.5).to(dtype)
        v = k[..., :E].clone() if latent_rows else torch.randn((c + q, Hk, E), generator=g).to(dtype)
        for j in range(c + q):
            kc[table[e, j // P], j % P] = k[j]
            if not latent_rows:
                vc[table[e, j // P], j % P] = v[j]
        ks.append(k.double().repeat_interleave(Hq // Hk, dim=1)); vs.append(v.double().repeat_interleave(Hq // Hk, dim=1))
        qs.append((torch.randn((q, Hq, D), generator=g) * 1.5).to(dtype))
    sink = (torch.randn(Hq, generator=g) + 1.0) if sink_on else None
    n = sum(q for _, q in ctx_new)
    q_all = torch.cat(qs).reshape(n, Hq * D).cuda()
    cu = torch.tensor([0, 45, 48, 49], dtype=torch.int32).cuda()
    start = torch.tensor([c for c, _ in ctx_new], dtype=torch.int32).cuda()
    out = torch.full((n, Hq * E), float("nan"), dtype=torch.float32 if kernel in ("simt", "general") else dtype).cuda()
    sk = None if sink is None else sink.cuda()
    common = (kc.cuda(), kc.cuda() if latent_rows else vc.cuda(), table.cuda(), cu, start)
    if kernel == "general":
        assert ops.attn_general_mma_supports(dtype, D, E)
        tpt = ops.attn_general_mma_tokens_per_tile(Hq, Hk)
        run = lambda work, **split: ops.attn_general_mma(q_all, Hq * D, out, *common, work, work.shape[0], Hq, Hk, scale,
                                                         window=code, sink=sk, **split)
    elif kernel == "equal":
        assert ops.attn_mma_supports(dtype, D)
        tpt = ops.attn_mma_tokens_per_tile(Hq, Hk)
        run = lambda work, **split: ops.attn_mma(q_all, Hq * D, out, *common, work, work.shape[0], Hq, Hk, D, code, scale, **split)
    elif kernel == "latent":
        assert ops.attn_latent_mma_supports(dtype, D, E)
        tpt = ops.attn_latent_mma_tokens_per_tile(Hq)
        run = lambda work, **split: ops.attn_latent_mma(q_all, Hq * D, out, common[0], *common[2:], work, work.shape[0], Hq, D, E,
                                                        scale, window=code, sink=sk, **split)
    else:
        tpt = ops.attn_simt_tokens_per_tile(Hq, Hk)
        run = lambda work, **split: ops.attn_simt(q_all, Hq * D, out, *common, work, work.shape[0], Hq, Hk, D, code, scale,
                                                  v_dim=E, sink=sk, **split)
    tiles = [(0, t) for t in range(0, 45, tpt)] + [(1, t) for t in range(0, 3, tpt)]
    run(torch.tensor(tiles, dtype=torch.int32).cuda())
    run(torch.tensor([(2, 0)], dtype=torch.int32).cuda(), split_size=64, n_splits=3)
    ops.check_status()
    got = out.cpu().double().view(n, Hq, E)
    tol = 2e-5 if name == "simt32" else 2.5e-2
    at = 0
    for e, (c, q) in enumerate(ctx_new):
        rows = gp.visible(c + q, window=window, chunk=chunk)[c:]
        sd = None if sink is None else sink.double()
        pad = torch.zeros((c, Hq, D), dtype=torch.float64)
        want = gp.softmax_attend(torch.cat([pad, qs[e].double()]), ks[e], vs[e], scale, gp.visible(c + q, window=window, chunk=chunk), sd)[c:]
        assert (got[at:at + q] - want).abs().max() < tol * max(1.0, want.abs().max().item()), f"entry {e}"
        if mask[1] < 100 and c + q > mask[1]:
            # the mask matters: one position more (a window of one more, a chunk that starts one earlier) changes the result
            wider = rows.clone()
            for i in range(q):
                first = int(torch.nonzero(rows[i])[0])
                if first > 0:
                    wider[i, first - 1] = True
            other = gp.softmax_attend(torch.cat([pad, qs[e].double()]), ks[e], vs[e], scale,
                                      torch.cat([gp.visible(c + q)[:c], wider]), sd)[c:]
            assert (other - want).abs().max() > 1e-3, f"entry {e}: the mask does not matter here"
        at += q


@pytest.mark.parametrize("mask", [("window", 1), ("window", 72), ("window", 200), ("chunk", 7), ("chunk", 120), ("chunk", 384),
                                  ("chunk", 100000)])
@pytest.mark.parametrize("Hq,Hk,sink_on", [(4, 2, False), (3, 3, True), (8, 1, True)])
def test_windows_and_chunks_on_the_tcgen05_prompt_kernel(Hq, Hk, sink_on, mask):
    """Whole 128-row tiles of a prompt portion on heads of 128 under a window or chunks: earlier context in the cache
    whose pages before the first visible key have been given back (no page in the table), a last tile that is not
    full, an entry that is exactly one tile from position 0; with and without a sink."""
    from jax_vllm_b200 import ops
    D, P, n_pages, scale = 128, 16, 64, 1.3 * 128 ** -0.5
    tpt = ops.attn_tcgen05_tokens_per_tile(Hq, Hk)
    ctx_new = [(300, 2 * tpt + 22), (0, tpt)]
    window = mask[1] if mask[0] == "window" else None
    chunk = mask[1] if mask[0] == "chunk" else None
    code = ops.mask_code(window, chunk)
    g = torch.Generator().manual_seed(Hq + mask[1])
    table = scrambled_pages(ctx_new, P, n_pages, g)
    kc = torch.full((n_pages, P, Hk, D), float("nan"), dtype=torch.bfloat16)
    vc = torch.full((n_pages, P, Hk, D), float("nan"), dtype=torch.bfloat16)
    ks, vs, qs = [], [], []
    for e, (c, q) in enumerate(ctx_new):
        k = (torch.randn((c + q, Hk, D), generator=g) * 1.5).to(torch.bfloat16)
        v = torch.randn((c + q, Hk, D), generator=g).to(torch.bfloat16)
        first_needed = int(torch.nonzero(gp.visible(c + q, window=window, chunk=chunk)[c])[0])     # of the entry's first query
        for j in range(c + q):
            if (j // P + 1) * P <= first_needed:
                table[e, j // P] = -1                       # the page went back to the pool
            else:
                kc[table[e, j // P], j % P], vc[table[e, j // P], j % P] = k[j], v[j]
        ks.append(k.double().repeat_interleave(Hq // Hk, dim=1)); vs.append(v.double().repeat_interleave(Hq // Hk, dim=1))
        qs.append((torch.randn((q, Hq, D), generator=g) * 1.5).to(torch.bfloat16))
    sink = (torch.randn(Hq, generator=g) + 2.0) if sink_on else None
    n = sum(q for _, q in ctx_new)
    q_all = torch.cat(qs).reshape(n, Hq * D).cuda()
    cu = torch.tensor([0, ctx_new[0][1], n], dtype=torch.int32).cuda()
    start = torch.tensor([c for c, _ in ctx_new], dtype=torch.int32).cuda()
    out = torch.full((n, Hq * D), float("nan"), dtype=torch.bfloat16).cuda()
    tiles = [(e, t) for e, (_, q) in enumerate(ctx_new) for t in range(0, q, tpt)]
    ops.attn_tcgen05(q_all, Hq * D, out, kc.cuda(), vc.cuda(), table.cuda(), cu, start,
                     torch.tensor(tiles, dtype=torch.int32).cuda(), len(tiles), Hq, Hk, D, scale,
                     sink=None if sink is None else sink.cuda(), window=code)
    ops.check_status()
    got = out.cpu().double().view(n, Hq, D)
    at = 0
    for e, (c, q) in enumerate(ctx_new):
        pad = torch.zeros((c, Hq, D), dtype=torch.float64)
        want = gp.softmax_attend(torch.cat([pad, qs[e].double()]), ks[e], vs[e], scale, gp.visible(c + q, window=window, chunk=chunk),
                                 None if sink is None else sink.double())[c:]
        assert (got[at:at + q] - want).abs().max() < 2.5e-2 * max(1.0, want.abs().max().item()), f"entry {e}"
        at += q


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,E,N,G,NG,taps", [(4, 8, 16, 2, 1, 3), (3, 8, 5, 3, 2, 2), (8, 16, 64, 1, 4, 4), (1, 6, 4, 1, 1, 1),
                                             (2, 64, 128, 2, 2, 4), (6, 10, 24, 3, 6, 4)])
def test_state_space_mixer_alone(H, E, N, G, NG, taps, dtype):
    """Convolution, step sizes, scan and gated group norm from a given projection: three entries of unequal length in
    slots given out of order, then a second call that carries on token by token and in a short portion; compared
    with the plain mixer run whole on each sequence (identity matrices for its two products)."""
    from jax_vllm_b200 import ops
    from jax_vllm_b200.config.model_spec import StateSpaceSpec
    from jax_vllm_b200.parts import BuildContext
    from jax_vllm_b200.parts.base import StateLayerCache, StepContext
    from jax_vllm_b200.parts.state_space import StateSpace
    g = torch.Generator().manual_seed(H * E + N)
    inner, rows_in = H * E, 2 * H * E + 2 * G * N + H
    mx = {"heads": H, "vdim": E, "state": N, "groups": G, "norm_groups": NG, "conv": taps}
    ch = inner + 2 * G * N
    w = {"l.m.in": torch.eye(rows_in), "l.m.o": torch.eye(inner), "l.m.conv": 0.5 * torch.randn((ch, taps), generator=g),
         "l.m.conv.b": 0.3 * torch.randn(ch, generator=g), "l.m.dt_bias": 0.5 * torch.randn(H, generator=g),
         "l.m.A_log": -1.0 + 0.5 * torch.randn(H, generator=g), "l.m.D": 1.0 + 0.2 * torch.randn(H, generator=g),
         "l.m.norm": 1.0 + 0.1 * torch.randn(inner, generator=g)}
    w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    part = StateSpace(StateSpaceSpec(rows_in, H, E, N, G, NG, taps, 1e-5, prefix="m"), "l", BuildContext(dtype, torch.device("cuda")))
    part.bind({k: v.to(torch.bfloat16).cuda() for k, v in w.items()})
    first, second, slots, n_slots = [70, 1, 9], [1, 5, 2], [3, 0, 4], 6
    seqs = [torch.randn((first[e] + second[e], rows_in), generator=g).to(dtype).float() for e in range(3)]
    need = part.cache_need()
    state = torch.zeros((n_slots,) + need.shape, dtype=torch.float32).cuda()
    state[2] = 5.0
    wd = {k: v.double() for k, v in w.items()}
    want = [gp.mamba2(s.double(), wd, "l.m", mx, 1e-5) for s in seqs]
    done = [0] * 3
    for lengths in (first, second):
        rows = torch.cat([seqs[e][done[e]:done[e] + n] for e, n in enumerate(lengths)]).to(dtype).cuda()
        cu, sl = entries_of(lengths, slots)
        step = StepContext(n_tokens=rows.shape[0], n_entries=3, token_ids=None, positions=None, token_entry=None, cu_seqlens=cu,
                           start_pos=None, state_slots=sl, logit_rows=None, n_logit_rows=0, block_tables=[], tile_work={},
                           decode_work=(None, 0), max_seq_len=0)
        out = torch.empty((rows.shape[0], inner), dtype=dtype).cuda()
        part.from_projection(rows, step, StateLayerCache(state), out)
        ops.check_status()
        at = 0
        for e, n in enumerate(lengths):
            ref = want[e][done[e]:done[e] + n]
            tol = 3e-5 if dtype == torch.float32 else 3e-2
            assert (out[at:at + n].double().cpu() - ref).abs().max() < tol * max(1.0, ref.abs().max().item()), (e, lengths)
            at += n
            done[e] += n
    assert bool((state[2] == 5.0).all()) and bool((state[1] == 0.0).all())


# ------------------------------------------------- whole models through the replay class
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt(setup, dtype, tmp_path):
    tag, folder, seqs, want = setup
    steps = whole("r0", seqs["r0"])
    replay(folder, tag, dtype, steps, tmp_path, max_tokens=256)
    compare(steps, tmp_path, CONFIGS[tag]["vocab"], want, dtype, case=f"gogivik {tag}, whole")


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_tokens_one_by_one(setup, dtype, graphs, tmp_path):
    tag, folder, seqs, want = setup
    steps = prefix_then_single("r1", seqs["r1"], tail=25)
    rep = replay(folder, tag, dtype, steps, tmp_path, max_tokens=128, cuda_graphs=graphs)
    compare(steps, tmp_path, CONFIGS[tag]["vocab"], want, dtype, case=f"gogivik {tag}, decoded")
    assert (rep.runner.graph_replays > 0) == graphs


@pytest.mark.parametrize("sizes", [(2,), (5, 1, 2, 19), (33, 3)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions(setup, dtype, sizes, tmp_path):
    tag, folder, seqs, want = setup
    steps = portions("r2", seqs["r2"], sizes)
    replay(folder, tag, dtype, steps, tmp_path, max_tokens=256)
    compare(steps, tmp_path, CONFIGS[tag]["vocab"], want, dtype, case=f"gogivik {tag}, portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_side_by_side_in_reused_pages_and_slots(setup, dtype, tmp_path):
    tag, folder, seqs, want = setup
    steps = mixed_trace(seqs)
    P = PAGE[tag]
    live3 = sum(sorted(-(-len(s) // P) * P for s in seqs.values())[-3:])
    rep = replay(folder, tag, dtype, steps, tmp_path, max_tokens=live3)
    compare(steps, tmp_path, CONFIGS[tag]["vocab"], want, dtype, case=f"gogivik {tag}, side by side")
    assert sum(m["pages_allocated"] for m in rep.records) > rep.cache.num_pages     # pages went out again


def test_schedules_agree_with_each_other_in_32_bit(setup, tmp_path):
    """A position's logits do not depend on the cut, the batch, the pages or the state slot beyond rounding."""
    tag, folder, seqs, _ = setup
    V = CONFIGS[tag]["vocab"]
    a = whole("r0", seqs["r0"])
    b = portions("r0", seqs["r0"], (5, 1, 2, 19))
    c = mixed_trace(seqs)
    replay(folder, tag, "float32", a, tmp_path / "a", 256)
    replay(folder, tag, "float32", b, tmp_path / "b", 256)
    replay(folder, tag, "float32", c, tmp_path / "c", 512)
    ga, gb, gc = (collect(s, tmp_path / d, V)["r0"] for s, d in ((a, "a"), (b, "b"), (c, "c")))
    for pos in ga:
        assert abs(ga[pos] - gb[pos]).max() < 1e-4 and abs(ga[pos] - gc[pos]).max() < 1e-4


def test_trace_run_program(tmp_path):
    """bin/trace_run as a program on a Gogivik folder: stdin steps, `done <step>` lines, files on disk, exit 0."""
    c = CONFIGS["gb"]
    weights = make_weights(c, seed=9)
    folder = write_folder(tmp_path / "model", c, weights)
    seqs = {f"r{i}": random_tokens(n, c["vocab"], seed=40 + i) for i, n in enumerate([40, 21, 33, 12, 18])}
    want = {rid: oracle(c, stored(weights), t) for rid, t in seqs.items()}
    steps = mixed_trace(seqs)
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
                           "--out", str(tmp_path / "out"), "--max-tokens", "192"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                          env=dict(os.environ), timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    compare(steps, tmp_path / "out", c["vocab"], want, "float32")


# ------------------------------------------------------- weights that make a fault show
def special(tmp_path, c, weights, tokens, dtype, sizes=None, page=16, tail=0):
    from jax_vllm_b200.engine.replay import Replayer
    folder = write_folder(tmp_path / "model", c, weights)
    if tail:
        steps = prefix_then_single("r", tokens, tail=tail)
    else:
        steps = whole("r", tokens) if sizes is None else portions("r", tokens, sizes)
    out = tmp_path / f"out_{dtype}_{sizes}_{tail}"
    rep = Replayer(folder, dtype, out, max_tokens=-(-len(tokens) // 64) * 64, page_size=page)
    rep.run_stream(json.dumps(s) for s in steps)
    return steps, out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_edges_of_chunks_and_windows_and_the_sink_show(dtype, tmp_path):
    """Sharp attention (queries and keys three times as large): a chunk or a window that is one position off, or a sink
    that is left out, moves the plain logits by far more than the limit; the engine agrees with the true ones whole,
    in portions that cut through chunks and windows, and decoding."""
    c = config(160, 64, [layer(attention(4, 2, 16, 24, chunk=24, rot_dims=8, factor=2.0), dense(48)),
                         layer(latent(4, 16, 8, 16, kv_rank=32, q_rank=24, window=13), None)], taps=3, logit_scale=1.0)
    weights = make_weights(c, seed=31)
    for name in ("l0.mix.q", "l0.mix.k", "l1.mix.uq", "l1.mix.uk"):
        weights[name] = 3.0 * weights[name]
    weights["l1.mix.sink"] = weights["l1.mix.sink"] + 2.0
    w = stored(weights)
    tokens = random_tokens(120, c["vocab"], seed=77)
    want = {"r": oracle(c, w, tokens)}
    lim = limits(dtype, want["r"])
    for change in ("chunk+", "chunk-", "window+", "window-", "sink"):
        other, w2 = copy.deepcopy(c), w
        if change.startswith("chunk"):
            other["layers"][0]["mixer"]["mask"]["size"] += 1 if change.endswith("+") else -1
        elif change.startswith("window"):
            other["layers"][1]["mixer"]["mask"]["size"] += 1 if change.endswith("+") else -1
        else:
            w2 = dict(w, **{"l1.mix.sink": w["l1.mix.sink"] - 60.0})
        assert (oracle(other, w2, tokens) - want["r"]).abs().max().item() > 20 * limits("float32", want["r"]), change
    for kw in (dict(), dict(sizes=(7, 2)), dict(sizes=(24, 13)), dict(tail=60)):
        steps, out = special(tmp_path, c, weights, tokens, dtype, **kw)
        compare(steps, out, c["vocab"], want, dtype)
    assert lim > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far", [0, 1, 63, 64, 200])
def test_a_token_far_back_in_the_state(far, dtype, tmp_path):
    """A state that forgets slowly (a small decay rate) over 330 tokens: another token at one far position moves the
    last logits by much more than the limit in the plain implementation, and the engine agrees with it whole (segments
    side by side), in portions and decoding."""
    c = config(120, 48, [layer(mamba(2, 12, 16, groups=1, norm_groups=1, conv=2), None)], taps=2)
    weights = make_weights(c, seed=41)
    weights["l0.mix.A_log"] = torch.full((2,), -7.0)
    w = stored(weights)
    tokens = random_tokens(330, c["vocab"], seed=78)
    want = {"r": oracle(c, w, tokens)}
    changed = list(tokens)
    changed[far] = (tokens[far] + 1) % c["vocab"]
    moved = (oracle(c, w, changed)[-1] - want["r"][-1]).abs().max().item()
    assert moved > 20 * limits("float32", want["r"])
    for kw in (dict(), dict(sizes=(64, 1, 70)), dict(tail=40)):
        steps, out = special(tmp_path, c, weights, tokens, dtype, **kw)
        compare(steps, out, c["vocab"], want, dtype)


# ----------------------------------------------------------- generation, scheduler, entry point
def plain_greedy(c, w, prompt, n):
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(gp.forward(c, w, seq)[-1].argmax()))
    return seq[len(prompt):]


def test_greedy_generation_through_the_entry_point(tmp_path):
    """make_driver + generate: the scheduler's portions, decode steps from captured graphs, sampling; 40 tokens each
    (decoding passes over the ends of chunks and windows)."""
    from jax_vllm_b200 import SamplingParams, generate, load_from_path, make_driver
    c = CONFIGS["ga"]
    weights = make_weights(c, seed=21)
    folder = write_folder(tmp_path / "model", c, weights)
    model = load_from_path(folder, dtype="fp32")
    d = make_driver(model, max_num_seqs=3, max_model_len=96, block_size=16, max_tokens_per_step=16)
    prompts = [random_tokens(n, c["vocab"], seed=50 + n) for n in (21, 5, 40)]
    got = generate(d, prompts, SamplingParams(max_new_tokens=40))
    assert got == [plain_greedy(c, stored(weights), p, 40) for p in prompts]
    assert d.runner.graph_replays > 0
    d.cache.check()


def test_random_arrivals_with_few_pages_and_slots(tmp_path):
    """Requests arrive at random steps into a pool too small for them: the youngest is preempted and run again, pages
    and state slots come back and are used again (a slot's state starts from zero for its next owner); greedy tokens
    depend on none of it."""
    import random
    from jax_vllm_b200 import SamplingParams, add_request, has_work, load_from_path, make_driver, step
    c = CONFIGS["gb"]
    weights = make_weights(c, seed=22)
    folder = write_folder(tmp_path / "model", c, weights)
    rng = random.Random(1)
    model = load_from_path(folder, dtype="fp32")
    d = make_driver(model, max_num_seqs=3, max_model_len=64, block_size=8, num_blocks=9, max_tokens_per_step=24)
    prompts = [random_tokens(rng.randrange(1, 30), c["vocab"], seed=100 + i) for i in range(8)]
    new_tokens = [rng.randrange(6, 27) for _ in prompts]
    waiting, ids = list(range(len(prompts))), {}
    while waiting or has_work(d):
        if waiting and (rng.random() < 0.4 or not has_work(d)):
            i = waiting.pop(0)
            ids[i] = add_request(d, prompts[i], SamplingParams(max_new_tokens=new_tokens[i]))
        step(d)
        d.cache.check()
    assert not d.cache.live
    w = stored(weights)
    for i, prompt in enumerate(prompts):
        assert d.requests[ids[i]].output_ids == plain_greedy(c, w, prompt, new_tokens[i]), f"request {i}"


def test_command_line(tmp_path):
    """cli.py as a user runs it on a Gogivik folder: prompts as token ids, 32-bit; the printed ids are the plain
    implementation's greedy tokens."""
    c = CONFIGS["gd"]
    weights = make_weights(c, seed=23)
    folder = write_folder(tmp_path / "model", c, weights)
    prompts = [random_tokens(37, c["vocab"], seed=60), random_tokens(37, c["vocab"], seed=60)[:33] + [5, 6], [9]]
    cmd = [sys.executable, str(ROOT / "cli.py"), "--model-path", str(folder), "--dtype", "fp32", "--max-tokens", "7",
           "--max-model-len", "128", "--block-size", "32", "--no-prewarm"]
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(map(str, p))]
    proc = subprocess.run(cmd, capture_output=True, text=True, env=dict(os.environ), timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = [json.loads(line)["output_ids"] for line in proc.stdout.splitlines() if line.startswith("{")]
    assert got == [plain_greedy(c, stored(weights), p, 7) for p in prompts]


# ------------------------------------------------------------------ configurations drawn at random
def random_configuration(seed):
    import random
    rng = random.Random(seed)
    width = rng.choice([40, 56, 72, 96])
    layers = []
    for _ in range(rng.randrange(2, 5)):
        kind = rng.choice(["attention", "latent", "mamba"])
        if kind == "attention":
            kv = rng.choice([1, 2, 3])
            dim, vdim = rng.choice([8, 12, 16, 32, 64]), rng.choice([6, 8, 16, 32, 64])
            mixer = attention(kv * rng.choice([1, 2, 3]), kv, dim, vdim, chunk=rng.randrange(1, 70),
                              rot_dims=rng.choice([2, dim // 2 // 2 * 2, dim]), base=rng.choice([1e3, 1e4, 1e6]),
                              factor=rng.choice([None, 1.0, 8.0]))
        elif kind == "latent":
            rot = rng.choice([2, 4, 8, 16])
            mixer = latent(rng.randrange(1, 6), rng.choice([4, 8, 16, 24]), rot, rng.choice([4, 8, 16, 24]),
                           kv_rank=rng.choice([8, 12, 16, 24, 48, 64]), q_rank=rng.choice([4, 8, 20]), window=rng.randrange(1, 70))
        else:
            groups = rng.choice([1, 2, 3])
            heads = groups * rng.choice([1, 2])
            mixer = mamba(heads, rng.choice([4, 6, 8, 16]), rng.choice([3, 8, 16, 32]), groups,
                          norm_groups=rng.choice([1, 2, heads]), conv=rng.randrange(1, 6))
        layers.append(layer(mixer, rng.choice([None, dense(rng.choice([8, 24, 40, 64]))])))
    return config(rng.randrange(60, 300), width, layers, eps=rng.choice([1e-6, 1e-5, 1e-4]), taps=rng.randrange(1, 6),
                  logit_scale=rng.choice([None, 0.5, 2.0]))


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(seed, tmp_path):
    """Layer orders, sizes and constants drawn at random: a prompt whole and in portions, and decoded, in both
    precisions; and five requests side by side in 32-bit."""
    c = random_configuration(seed)
    for ly in c["layers"]:                      # values that a state-space norm can split evenly
        mx = ly["mixer"]
        if ly["type"] == "mamba2" and (mx["heads"] * mx["vdim"]) % mx["norm_groups"]:
            mx["norm_groups"] = 1
    weights = make_weights(c, seed=60 + seed, up_scale=0.75)      # narrow layers: squares of large numbers would set the bfloat16 error
    folder = write_folder(tmp_path / "model", c, weights)
    w = stored(weights)
    page = [4, 8, 16, 32][seed % 4]
    seqs = {f"r{i}": random_tokens(n, c["vocab"], seed=200 + 10 * seed + i) for i, n in enumerate([90, 33, 61, 12, 40])}
    want = {rid: oracle(c, w, t) for rid, t in seqs.items()}
    rounding = {rid: rounding_error(c, w, seqs[rid]) for rid in ("r0", "r2")}
    from jax_vllm_b200.engine.replay import Replayer
    for dtype in ("float32", "bfloat16"):
        for k, steps in enumerate((whole("r0", seqs["r0"]), portions("r0", seqs["r0"], (3, 1, 30, 2)),
                                   prefix_then_single("r2", seqs["r2"], tail=22))):
            out = tmp_path / f"{dtype}_{k}"
            rep = Replayer(folder, dtype, out, max_tokens=128, page_size=page)
            rep.run_stream(json.dumps(s) for s in steps)
            compare(steps, out, c["vocab"], want, dtype, rounding=rounding)
    steps = mixed_trace(seqs)
    rep = Replayer(folder, "float32", tmp_path / "mixed", max_tokens=320, page_size=page)
    rep.run_stream(json.dumps(s) for s in steps)
    rep.cache.check()
    compare(steps, tmp_path / "mixed", c["vocab"], want, "float32")
