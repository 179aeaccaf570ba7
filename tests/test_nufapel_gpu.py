"""The Nufapel design in the engine against the plain implementation (tests/plain/nufapel_plain.py): every mechanism
alone, then models of several sizes through the replay program's class (whole, last tokens one by one, portions down
to two tokens, unequal requests side by side in reused pages and state slots), special weights where random ones would
hide a fault, and greedy generation through the entry point and its scheduler."""

from __future__ import annotations

import json
import math
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from tests.nufapel_util import (CONFIGS, PAGE, config, delta, dense, layer, make_weights, moe, pair, stored,
                                write_folder)
from tests.plain import nufapel_plain as npl
from tests.test_replay_gpu import limits
from tests.util import collect, portions, prefix_then_single, random_tokens, whole

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
LENGTHS = {"na": [70, 45, 100, 33, 52], "nb": [90, 38, 64, 51, 27], "nc": [200, 70, 150, 40, 66], "nd": [61, 40, 83, 35, 20],
           "ne": [170, 60, 100, 37, 45]}
CLOSE_CALL = 0.02      # a difference of router scores below which bfloat16 may choose another expert
EXCUSED = 0.25         # share of the positions that may differ for that reason


def oracle(c, w, tokens):
    """(logits, the first position whose routing is a close call in some layer, or a huge number)."""
    margins = []
    logits = npl.forward(c, w, tokens, margins=margins).to(torch.float32)
    close = [int(torch.nonzero(m < CLOSE_CALL)[0]) for m in margins if bool((m < CLOSE_CALL).any())]
    return logits, min(close) if close else 1 << 30


def compare(steps, out_dir, vocab, want, dtype, case=None, close=None):
    """Every written row against the oracle's.  32-bit holds every position and the greedy token.  In bfloat16 one
    position in fifty (or one) may be over the limit by up to half of it, and a position at or after a token whose
    choice of experts hangs on a small difference of scores (`close`: request -> first such position) is excused,
    as long as no more than EXCUSED of all positions are."""
    from tests.conftest import record_worst
    got = collect(steps, out_dir, vocab)
    worst, lim_of_worst, total, slightly, excused = 0.0, 0.0, 0, 0, 0
    for rid, rows in got.items():
        lim = limits(dtype, want[rid])
        first_close = (close or {}).get(rid, 1 << 30) if dtype != "float32" else 1 << 30
        for pos, row in rows.items():
            total += 1
            w = want[rid][pos]
            diff = (torch.from_numpy(row.copy()) - w).abs().max().item()
            assert math.isfinite(diff), f"{rid} position {pos}: not a number"
            if diff > lim and pos >= first_close:
                excused += 1
                continue
            if dtype != "float32" and lim < diff <= 1.5 * lim:
                slightly += 1
                continue
            assert diff <= lim, f"{rid} position {pos}: |diff| {diff:.3e} > {lim:.3e}"
            if diff >= worst:
                worst, lim_of_worst = diff, lim
            if dtype == "float32":
                top2 = w.topk(2).values
                assert int(row.argmax()) == int(w.argmax()) or float(top2[0] - top2[1]) < 1e-4
    assert slightly <= max(1, 0.02 * total), f"{slightly} of {total} positions are over the limit"
    assert excused <= EXCUSED * total, f"{excused} of {total} positions differ after a close call of the router"
    if case is not None:
        record_worst(case, dtype, worst, lim_of_worst)
    return got


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def setup(request, tmp_path_factory):
    tag = request.param
    c = CONFIGS[tag]
    weights = make_weights(c, seed=5)
    folder = write_folder(tmp_path_factory.mktemp(f"nufapel_{tag}"), c, weights)
    w = stored(weights)
    seqs = {f"r{i}": random_tokens(n, c["vocab"], seed=20 + i) for i, n in enumerate(LENGTHS[tag])}
    want, close = {}, {}
    for rid, t in seqs.items():
        want[rid], close[rid] = oracle(c, w, t)
    assert all(v.abs().max() > 1.0 for v in want.values())     # logits of order one, not a flat model
    return tag, folder, seqs, want, close


def replay(folder, tag, dtype, steps, out_dir, max_tokens, **switches):
    from jax_vllm_b200.engine.replay import Replayer
    rep = Replayer(folder, dtype, out_dir, max_tokens=max_tokens, page_size=PAGE[tag], **switches)
    rep.run_stream(json.dumps(s) for s in steps)
    rep.cache.check()
    assert not rep.cache.live
    return rep


# ------------------------------------------------------------------ mechanisms alone
def entries_of(lengths, slots, n_slots):
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32).cuda()
    return cu, torch.tensor(slots, dtype=torch.int32).cuda()


@pytest.mark.parametrize("segment", [0, 4, 7])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,V", [(2, 16, 16), (3, 20, 20), (1, 40, 40), (2, 64, 64), (1, 128, 128), (2, 7, 7), (1, 200, 200)])
def test_delta_rule_alone(H, D, V, dtype, segment):
    """The prepare kernel and the scan with the removal term: three entries of unequal length (one of a single
    token) whose states start from random matrices in slots given out of order; a second call carries on from what
    the first left, token by token, and an unused slot stays as it was.  `segment` > 0: the entries run in segments
    of so many tokens side by side (23 tokens: whole segments and a rest; 9: one token more than two of 4)."""
    from jax_vllm_b200 import ops
    g = torch.Generator().manual_seed(H * D)
    lengths, slots, n_slots = [23, 1, 9], [3, 0, 4], 6
    n = sum(lengths)
    cols = 3 * H * D + 5
    proj = torch.randn((n, cols), generator=g).to(dtype)
    r_off, k_off, a_off = 0, H * D + 5, 2 * H * D + 5
    zw = (2.0 * torch.randn((n, H * D), generator=g)).to(dtype)
    vrow = torch.randn((n, H * V + 3), generator=g).to(dtype)
    a_bias, w_bias = (0.3 * torch.randn(H * D, generator=g)).bfloat16(), (0.3 * torch.randn(H * D, generator=g)).bfloat16()
    state0 = torch.randn((n_slots, H * D * V + 11), generator=g)
    state = state0.clone().cuda()
    cu, sl = entries_of(lengths, slots, n_slots)
    packed = ops.delta_prepare(proj.cuda(), r_off, k_off, a_off, zw.cuda(), a_bias.cuda(), w_bias.cuda(), H, D)
    o = ops.state_scan(packed, vrow.cuda(), 3, state, cu, sl, len(lengths), V, segment=segment)
    ops.check_status()
    p64 = proj.double()
    r, k = p64[:, r_off:r_off + H * D].view(n, H, D), p64[:, k_off:k_off + H * D].view(n, H, D)
    a = torch.sigmoid(p64[:, a_off:a_off + H * D] + a_bias.double()).view(n, H, D)
    w = npl.delta_decay(zw.double() + w_bias.double()).view(n, H, D)
    v = vrow.double()[:, 3:3 + H * V].view(n, H, V)
    tol = 2e-4 if dtype == torch.float32 else 2e-3                  # the recurrence is 32-bit in both
    at, after = 0, {}
    for e, T in enumerate(lengths):
        S0 = state0[slots[e], :H * D * V].double().view(H, D, V)
        want, S = npl.delta_scan(r[at:at + T], k[at:at + T], v[at:at + T], w[at:at + T], a[at:at + T], S0)
        got = o[at:at + T].cpu().double().view(T, H, V)
        assert (got - want).abs().max() < tol * max(1.0, want.abs().max().item()), f"entry {e}"
        after[slots[e]] = S
        assert (state[slots[e], :H * D * V].cpu().double().view(H, D, V) - S).abs().max() < tol * max(1.0, S.abs().max().item())
        at += T
    left = [s for s in range(n_slots) if s not in slots]
    assert torch.equal(state[left].cpu(), state0[left]) and torch.equal(state[:, H * D * V:].cpu(), state0[:, H * D * V:])
    # one more token for entries 0 and 2 only, in the other order: decoding from the carried state
    cu2, sl2 = entries_of([1, 1], [slots[2], slots[0]], n_slots)
    packed2 = packed[[n - 1, 0]].contiguous()
    v2 = vrow[[n - 1, 0]].cuda()
    o2 = ops.state_scan(packed2, v2, 3, state, cu2, sl2, 2, V)
    for row, (tok, slot) in enumerate(((n - 1, slots[2]), (0, slots[0]))):
        want, _ = npl.delta_scan(r[tok:tok + 1], k[tok:tok + 1], v[tok:tok + 1], w[tok:tok + 1], a[tok:tok + 1], after[slot])
        assert (o2[row].cpu().double().view(1, H, V) - want).abs().max() < tol * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("segment", [0, 5, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,V,cap", [(2, 8, 24, 15.0), (3, 20, 12, 8.0), (1, 36, 28, 4.0), (2, 128, 64, 15.0),
                                       (1, 12, 6, 30.0), (1, 256, 40, 15.0), (4, 32, 32, 2.0), (1, 16, 31, 6.0)])
def test_matrix_memory_alone(H, D, V, cap, dtype, segment):
    """The gate scan (normaliser and running maximum) and the matrix scan: entries of unequal length from states that
    are zero (a fresh request: the maximum starts at 0) or carried, gates pushed to both sides of their cap."""
    from jax_vllm_b200 import ops
    g = torch.Generator().manual_seed(H * D + V)
    lengths, slots, n_slots = [17, 1, 30], [2, 5, 1], 6
    n = sum(lengths)
    q_off, k_off, v_off, i_off, f_off = 0, H * D, 2 * H * D, 2 * H * D + H * V + 2, 2 * H * D + H * V + 2 + H
    proj = torch.randn((n, f_off + H + 1), generator=g)
    proj[:, i_off:i_off + 2 * H] *= 6.0                     # pre-activations well beyond small caps
    proj = proj.to(dtype)
    i_bias, f_bias = (torch.randn(H, generator=g)).bfloat16(), (2.0 + torch.randn(H, generator=g)).bfloat16()
    mats = H * D * V
    width = mats + H * D + H
    state0 = torch.zeros((n_slots, width))
    state0[slots[2]] = torch.randn(width, generator=g)      # entry 2 carries on from an earlier portion
    state0[slots[2], mats + H * D:] = torch.tensor([1.5, -0.5, 0.3, 2.0][:H])
    state0[4] = 7.0                                         # a slot that no entry holds
    state = state0.clone().cuda()
    cu, sl = entries_of(lengths, slots, n_slots)
    packed, gates = ops.memory_gates(proj.cuda(), q_off, k_off, i_off, f_off, i_bias.cuda(), f_bias.cuda(), cap, D ** -0.5,
                                     state[:, mats + H * D:], cu, sl, len(lengths), H, D)
    o = ops.state_scan(packed, proj.cuda(), v_off, state, cu, sl, len(lengths), V, state_n=state[:, mats:mats + H * D],
                       gates=gates, segment=segment)
    ops.check_status()
    # the scan leaves n . q and the running maximum in `gates`; the division by max(|n . q|, exp(-m)) + 1e-6 belongs
    # to the kernel that norms the heads (checked with it below) and is done here by hand
    den = torch.maximum(gates[:, :, 3].abs(), torch.exp(-gates[:, :, 2])) + 1e-6
    o = (o.view(n, H, V) / den[:, :, None]).reshape(n, H * V)
    p64 = proj.double()
    q = p64[:, q_off:q_off + H * D].view(n, H, D) * D ** -0.5
    k = p64[:, k_off:k_off + H * D].view(n, H, D)
    v = p64[:, v_off:v_off + H * V].view(n, H, V)
    gi, gf = npl.capped_gates(p64[:, i_off:i_off + H] + i_bias.double(), p64[:, f_off:f_off + H] + f_bias.double(), cap)
    tol = 3e-4 if dtype == torch.float32 else 3e-3
    at = 0
    for e, T in enumerate(lengths):
        row = state0[slots[e]].double()
        st = (row[:mats].view(H, D, V), row[mats:mats + H * D].view(H, D), row[mats + H * D:])
        want, (S, nn, m) = npl.memory_scan(q[at:at + T], k[at:at + T], v[at:at + T], gi[at:at + T], gf[at:at + T], st)
        got = o[at:at + T].cpu().double().view(T, H, V)
        assert (got - want).abs().max() < tol * max(1.0, want.abs().max().item()), f"entry {e}"
        new = state[slots[e]].cpu().double()
        assert (new[:mats].view(H, D, V) - S).abs().max() < tol * max(1.0, S.abs().max().item())
        assert (new[mats:mats + H * D].view(H, D) - nn).abs().max() < tol * max(1.0, nn.abs().max().item())
        assert (new[mats + H * D:] - m).abs().max() < 1e-5 * max(1.0, m.abs().max().item())
        at += T
    assert torch.equal(state[[0, 3, 4]].cpu(), state0[[0, 3, 4]])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_norm_and_pair_norm_alone(dtype):
    from jax_vllm_b200 import ops
    g = torch.Generator().manual_seed(3)
    n, H, V, eps = 7, 3, 20, 1e-5
    o = torch.randn((n, H * V), generator=g) * torch.tensor([1e-3, 1.0, 50.0]).repeat_interleave(V)   # heads of very different size
    weight = (1 + 0.1 * torch.randn(H * V, generator=g)).bfloat16()
    wide = torch.randn((n, H * V + 9), generator=g).to(dtype)
    out = torch.full((n, H * V + 4), float("nan"), dtype=dtype).cuda()
    ops.head_norm_gate(o.cuda(), weight.cuda(), wide.cuda()[:, 9:], out[:, 4:], H, V, eps)
    want = (npl.unit(o.double().view(n, H, V), eps).reshape(n, H * V) * weight.double()) * torch.sigmoid(wide.double()[:, 9:])
    tol = 2e-6 if dtype == torch.float32 else 2e-2
    assert (out[:, 4:].cpu().double() - want).abs().max() < tol * want.abs().max() and torch.isnan(out[:, :4]).all()
    # a matrix memory's heads are first divided by max(|n . q|, exp(-m)) + 1e-6: both branches of the maximum
    gates = torch.randn((n, H, 4), generator=g)
    gates[:, 0, 3] *= 30.0
    gates[:, 1, 2] += 5.0
    ops.head_norm_gate(o.cuda(), weight.cuda(), None, out[:, 4:], H, V, eps, gates=gates.cuda())
    den = torch.maximum(gates[:, :, 3].double().abs(), torch.exp(-gates[:, :, 2].double())) + 1e-6
    want = npl.unit(o.double().view(n, H, V) / den[:, :, None], eps).reshape(n, H * V) * weight.double()
    assert (out[:, 4:].cpu().double() - want).abs().max() < tol * want.abs().max()
    a, b = (torch.randn((n, 72), generator=g) * 3).to(dtype), (torch.randn((n, 72), generator=g) * 0.01).to(dtype)
    wa, wb = (1 + 0.1 * torch.randn(72, generator=g)).bfloat16(), (1 + 0.1 * torch.randn(72, generator=g)).bfloat16()
    got = ops.norm_mean2(a.cuda(), b.cuda(), wa.cuda(), wb.cuda(), 3e-6, 0.5)
    want = 0.5 * (npl.unit(a.double(), 3e-6) * wa.double() + npl.unit(b.double(), 3e-6) * wb.double())
    assert got.dtype == torch.float32 and (got.cpu().double() - want).abs().max() < 2e-6 * 4


def scrambled_pages(ctx_new, P, n_pages, g):
    """A block table over pages in a random order for entries of (cached, new) tokens."""
    width = max(-(-(c + q) // P) for c, q in ctx_new)
    table = torch.full((len(ctx_new), width), -1, dtype=torch.int32)
    free = torch.randperm(n_pages, generator=g).tolist()
    for e, (c, q) in enumerate(ctx_new):
        for i in range(-(-(c + q) // P)):
            table[e, i] = free.pop()
    return table


SINK_CASES = {
    # name: (query heads, key heads, key size, value size, rows of the bias table, largest distance, sink offset)
    "grouped_values_narrower": (6, 3, 32, 16, 8, 30, 0.0),
    "one_head_long_table": (1, 1, 64, 64, 32, 100, 2.0),
    "wide_group_saturating_early": (8, 1, 16, 48, 4, 5, -1.0),
    "heads_of_128": (4, 2, 128, 128, 16, 64, 4.0),
}


@pytest.mark.parametrize("kernel", ["simt32", "simt16", "mma16"])
@pytest.mark.parametrize("name", sorted(SINK_CASES))
def test_attention_with_temperature_distance_bias_and_sink_alone(name, kernel):
    """Both attention kernels with a temperature per head, a bias by bucketed distance and a sink: a prompt portion over
    several tiles behind earlier context (distances beyond the table's largest), a short prompt from position 0, and
    a single token whose keys are split into ranges that are merged with the sink counted once."""
    from jax_vllm_b200 import ops
    Hq, Hk, D, E, B, far, sink_shift = SINK_CASES[name]
    dtype = torch.float32 if kernel == "simt32" else torch.bfloat16
    g = torch.Generator().manual_seed(Hq * D + E + B)
    P, n_pages, scale = 8, 64, 1.3 * D ** -0.5
    ctx_new = [(37, 45), (0, 3), (130, 1)]
    table = scrambled_pages(ctx_new, P, n_pages, g)
    kc = torch.full((n_pages, P, Hk, D), float("nan"), dtype=dtype)
    vc = torch.full((n_pages, P, Hk, E), float("nan"), dtype=dtype)
    ks, vs, qs = [], [], []
    for e, (c, q) in enumerate(ctx_new):
        k = (torch.randn((c + q, Hk, D), generator=g) * 1.5).to(dtype)
        v = torch.randn((c + q, Hk, E), generator=g).to(dtype)
        for j in range(c + q):
            kc[table[e, j // P], j % P], vc[table[e, j // P], j % P] = k[j], v[j]
        ks.append(k.double().repeat_interleave(Hq // Hk, dim=1)); vs.append(v.double().repeat_interleave(Hq // Hk, dim=1))
        qs.append((torch.randn((q, Hq, D), generator=g) * 1.5).to(dtype))
    temp = 1.0 + 0.5 * torch.randn(Hq, generator=g)
    rel = 2.0 * torch.randn((B, Hq), generator=g)
    sink = torch.randn(Hq, generator=g) + sink_shift
    by_distance = torch.stack([rel[npl.distance_bucket(n, B, far)] for n in range(far + 1)], dim=1).contiguous()   # [Hq, far + 1]
    n = sum(q for _, q in ctx_new)
    q_all = torch.cat(qs).reshape(n, Hq * D).cuda()
    cu = torch.tensor([0, 45, 48, 49], dtype=torch.int32).cuda()
    start = torch.tensor([c for c, _ in ctx_new], dtype=torch.int32).cuda()
    out = torch.full((n, Hq * E), float("nan"), dtype=torch.float32).cuda()
    extra = dict(head_scale=temp.cuda(), dist_bias=by_distance.cuda(), sink=sink.cuda())
    common = (kc.cuda(), vc.cuda(), table.cuda(), cu, start)
    if kernel == "mma16":
        assert ops.attn_general_mma_supports(dtype, D, E)
        tpt = ops.attn_general_mma_tokens_per_tile(Hq, Hk)
        run = lambda work, **split: ops.attn_general_mma(q_all, Hq * D, out, *common, work, work.shape[0], Hq, Hk, scale, **split, **extra)
    else:
        tpt = ops.attn_simt_tokens_per_tile(Hq, Hk)
        run = lambda work, **split: ops.attn_simt(q_all, Hq * D, out, *common, work, work.shape[0], Hq, Hk, D, 0, scale,
                                                  v_dim=E, **split, **extra)
    tiles = [(0, t) for t in range(0, 45, tpt)] + [(1, t) for t in range(0, 3, tpt)]
    run(torch.tensor(tiles, dtype=torch.int32).cuda())
    run(torch.tensor([(2, 0)], dtype=torch.int32).cuda(), split_size=64, n_splits=3)
    ops.check_status()
    got = out.cpu().double().view(n, Hq, E)
    tol = 2e-5 if kernel == "simt32" else 2.5e-2
    at = 0
    for e, (c, q) in enumerate(ctx_new):
        want = npl.biased_sink_attend(qs[e].double(), ks[e], vs[e], scale, temp.double(), rel.double(), far, sink.double(), first=c)
        assert (got[at:at + q] - want).abs().max() < tol * max(1.0, want.abs().max().item()), f"entry {e}"
        # the parts matter: without the sink, or with a table that saturates one position earlier, the result differs
        no_sink = npl.biased_sink_attend(qs[e].double(), ks[e], vs[e], scale, temp.double(), rel.double(), far, sink.double() - 50.0, first=c)
        assert kernel != "simt32" or (no_sink - want).abs().max() > 20 * tol
        at += q


@pytest.mark.parametrize("Hq,Hk,B,far", [(4, 2, 16, 64), (3, 3, 32, 500), (8, 1, 6, 9)])
def test_temperature_distance_bias_and_sink_on_the_tcgen05_kernel(Hq, Hk, B, far):
    """Whole 128-row tiles of a prompt portion on heads of 128: earlier context in the cache (distances on both sides of
    the table's largest), a last tile that is not full, an entry that is exactly one tile; one head's temperature is
    negative (its largest score is then not its largest product)."""
    from jax_vllm_b200 import ops
    D, P, n_pages, scale = 128, 16, 40, 128 ** -0.5
    tpt = ops.attn_tcgen05_tokens_per_tile(Hq, Hk)
    ctx_new = [(100, 2 * tpt + 22), (0, tpt)]
    g = torch.Generator().manual_seed(Hq + B)
    table = scrambled_pages(ctx_new, P, n_pages, g)
    kc = torch.full((n_pages, P, Hk, D), float("nan"), dtype=torch.bfloat16)
    vc = torch.full((n_pages, P, Hk, D), float("nan"), dtype=torch.bfloat16)
    ks, vs, qs = [], [], []
    for e, (c, q) in enumerate(ctx_new):
        k = (torch.randn((c + q, Hk, D), generator=g) * 1.5).to(torch.bfloat16)
        v = torch.randn((c + q, Hk, D), generator=g).to(torch.bfloat16)
        for j in range(c + q):
            kc[table[e, j // P], j % P], vc[table[e, j // P], j % P] = k[j], v[j]
        ks.append(k.double().repeat_interleave(Hq // Hk, dim=1)); vs.append(v.double().repeat_interleave(Hq // Hk, dim=1))
        qs.append((torch.randn((q, Hq, D), generator=g) * 1.5).to(torch.bfloat16))
    temp = 1.0 + 0.4 * torch.randn(Hq, generator=g)
    temp[Hq - 1] = -0.7
    rel = 2.0 * torch.randn((B, Hq), generator=g)
    sink = torch.randn(Hq, generator=g) + 3.0
    by_distance = torch.stack([rel[npl.distance_bucket(n, B, far)] for n in range(far + 1)], dim=1).contiguous()
    n = sum(q for _, q in ctx_new)
    q_all = torch.cat(qs).reshape(n, Hq * D).cuda()
    cu = torch.tensor([0, ctx_new[0][1], n], dtype=torch.int32).cuda()
    start = torch.tensor([c for c, _ in ctx_new], dtype=torch.int32).cuda()
    out = torch.full((n, Hq * D), float("nan"), dtype=torch.bfloat16).cuda()
    tiles = [(e, t) for e, (_, q) in enumerate(ctx_new) for t in range(0, q, tpt)]
    ops.attn_tcgen05(q_all, Hq * D, out, kc.cuda(), vc.cuda(), table.cuda(), cu, start,
                     torch.tensor(tiles, dtype=torch.int32).cuda(), len(tiles), Hq, Hk, D, scale,
                     head_scale=temp.cuda(), dist_bias=by_distance.cuda(), sink=sink.cuda())
    ops.check_status()
    got = out.cpu().double().view(n, Hq, D)
    at = 0
    for e, (c, q) in enumerate(ctx_new):
        want = npl.biased_sink_attend(qs[e].double(), ks[e], vs[e], scale, temp.double(), rel.double(), far, sink.double(), first=c)
        assert (got[at:at + q] - want).abs().max() < 2.5e-2 * max(1.0, want.abs().max().item()), f"entry {e}"
        at += q


def test_norm_gate_router_and_experts_alone():
    """The dynamic-tanh norm with the gated sum in its pass, the router with sigmoid scores and groups that score as
    the sum of their two best, the clamped gated activation and the logit cap, each against its formula."""
    from jax_vllm_b200 import ops
    g = torch.Generator().manual_seed(4)
    n, W = 9, 52
    h0 = torch.randn((n, W), generator=g) * 3
    y = torch.randn((n, W), generator=g).bfloat16()
    z = torch.randn((n, W + 6), generator=g).bfloat16()
    zb, weight, bias = (torch.randn(W, generator=g).bfloat16() for _ in range(3))
    h = h0.clone().cuda()
    x = ops.gated_add_dyt(h, ops.GatedDelta(y.cuda(), z.cuda()[:, 6:], zb.cuda()), 0.6, weight.cuda(), bias.cuda(), torch.float32)
    want_h = h0.double() + torch.sigmoid(z.double()[:, 6:] + zb.double()) * y.double()
    assert (h.cpu().double() - want_h).abs().max() < 1e-5
    assert (x.cpu().double() - (torch.tanh(0.6 * want_h) * weight.double() + bias.double())).abs().max() < 1e-5
    for E, top, groups, keep, scale in ((12, 3, 4, 2, 1.5), (5, 2, 5, 3, 2.0), (8, 4, 1, 1, 0.5), (6, 1, 3, 1, 1.0), (9, 3, 3, 3, 1.0)):
        logits = torch.randn((40, E), generator=g) * 2
        ids, wts = ops.moe_route(logits.cuda(), top, groups, keep, True, scoring="sigmoid", group_score="top2_sum",
                                 renorm_eps=1e-20, weight_scale=scale)
        want_ids, want_w = npl.route(logits.double(), top, groups, keep, scale)
        order = ids.cpu().long().sort(dim=1)
        worder = want_ids.sort(dim=1)
        assert torch.equal(order.values, worder.values), (E, top, groups, keep)
        assert (wts.cpu().double().gather(1, order.indices) - want_w.gather(1, worder.indices)).abs().max() < 1e-6
    gu = (torch.randn((7, 2 * 24), generator=g) * 3).bfloat16()
    act = ops.glu_clamped(gu.cuda(), 2.0).cpu().double()
    gate, up = gu.double()[:, :24].clamp(max=2.0), gu.double()[:, 24:].clamp(-2.0, 2.0)
    want = gate * torch.sigmoid(1.702 * gate) * (up + 1.0)
    assert (act - want).abs().max() < 2e-2 * want.abs().max()
    lg = torch.randn((4, 33), generator=g) * 40
    assert (ops.softcap_(lg.clone().cuda(), 25.0).cpu().double() - 25.0 * torch.tanh(lg.double() / 25.0)).abs().max() < 1e-4


# ------------------------------------------------- whole models through the replay class
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt(setup, dtype, tmp_path):
    tag, folder, seqs, want, close = setup
    steps = whole("r0", seqs["r0"])
    replay(folder, tag, dtype, steps, tmp_path, max_tokens=256)
    compare(steps, tmp_path, CONFIGS[tag]["vocab"], want, dtype, case=f"nufapel {tag}, whole", close=close)


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_tokens_one_by_one(setup, dtype, graphs, tmp_path):
    tag, folder, seqs, want, close = setup
    steps = prefix_then_single("r1", seqs["r1"], tail=20)
    rep = replay(folder, tag, dtype, steps, tmp_path, max_tokens=128, cuda_graphs=graphs)
    compare(steps, tmp_path, CONFIGS[tag]["vocab"], want, dtype, case=f"nufapel {tag}, decoded", close=close)
    assert (rep.runner.graph_replays > 0) == graphs


@pytest.mark.parametrize("sizes", [(2,), (5, 1, 2, 19), (33, 3)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions(setup, dtype, sizes, tmp_path):
    tag, folder, seqs, want, close = setup
    steps = portions("r2", seqs["r2"], sizes)
    replay(folder, tag, dtype, steps, tmp_path, max_tokens=256)
    compare(steps, tmp_path, CONFIGS[tag]["vocab"], want, dtype, case=f"nufapel {tag}, portions", close=close)


def mixed_trace(seqs):
    """Five requests, never more than three live: portions of some beside single tokens of others; r3 starts only after
    r1 has ended and r4 after r0, in the pages and the state slots that those gave back; r1 is left out of a step and
    goes on later."""
    plan = [{"r0": 9, "r1": 2}, {"r0": 1, "r1": 17, "r2": 30}, {"r0": 30, "r2": 1}, {"r0": 1, "r1": 1, "r2": 2},
            {"r0": 1, "r1": 999, "r2": 1}, {"r0": 999, "r2": 40, "r3": 3}, {"r2": 999, "r3": 1, "r4": 5},
            {"r3": 2, "r4": 1}, {"r3": 999, "r4": 999}]
    fed = {r: 0 for r in seqs}
    steps = []
    for k, row in enumerate(plan):
        entries = []
        for rid, n in row.items():
            part = seqs[rid][fed[rid]:fed[rid] + n]
            if part:
                entries.append({"id": rid, "tokens": part, "want": list(range(len(part)))})
                fed[rid] += len(part)
        steps.append({"step": k, "entries": entries, "end": [e["id"] for e in entries if fed[e["id"]] == len(seqs[e["id"]])]})
    assert all(fed[r] == len(seqs[r]) for r in seqs)
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_side_by_side_in_reused_pages_and_slots(setup, dtype, tmp_path):
    tag, folder, seqs, want, close = setup
    steps = mixed_trace(seqs)
    P = PAGE[tag]
    live3 = sum(sorted(-(-len(s) // P) * P for s in seqs.values())[-3:])
    rep = replay(folder, tag, dtype, steps, tmp_path, max_tokens=live3)
    compare(steps, tmp_path, CONFIGS[tag]["vocab"], want, dtype, case=f"nufapel {tag}, side by side", close=close)
    paged = [g for g in rep.cache.groups if getattr(g, "pool", None) is not None]
    assert sum(m["pages_allocated"] for m in rep.records) > rep.cache.num_pages * max(1, len(paged))   # pages went out again


def test_schedules_agree_with_each_other_in_32_bit(setup, tmp_path):
    """A position's logits do not depend on the cut, the batch, the pages or the state slot beyond rounding."""
    tag, folder, seqs, _, _ = setup
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
    """bin/trace_run as a program on a Nufapel folder: stdin steps, `done <step>` lines, files on disk, exit 0."""
    c = CONFIGS["nb"]
    weights = make_weights(c, seed=9)
    folder = write_folder(tmp_path / "model", c, weights)
    seqs = {f"r{i}": random_tokens(n, c["vocab"], seed=40 + i) for i, n in enumerate([40, 21, 33, 12, 18])}
    want = {rid: npl.forward(c, stored(weights), t).to(torch.float32) for rid, t in seqs.items()}
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
def test_the_bias_tables_edges_the_sink_and_the_temperature_show(dtype, tmp_path):
    """An attention layer with sharp scores, a bias table of large entries that saturates at distance 23 and a heavy
    sink, over 90 tokens (most keys beyond the saturation, the steps of the buckets in between): moving the
    saturation by one position, dropping the sink or the temperature changes the plain logits greatly, and the engine
    equals the plain result whole, in portions down to two tokens and decoded."""
    c = config(70, 48, [layer(pair(4, 2, 16, 8, 1, 8, 8, bias_max=23, buckets=10), None)], eps=1e-6, softcap=40.0)
    w = make_weights(c, seed=31)
    w["l0.mix.left.q"] *= 2.0
    w["l0.mix.left.rel"] *= 4.0
    w["l0.mix.left.sink"] += 3.0
    w["l0.mix.left.temp"][:] = torch.tensor([1.6, 0.4, -0.8, 1.0])          # also a negative one
    w["l0.mix.right.out"] *= 0.05                                             # the attention side carries the layer
    tokens = random_tokens(90, 70, seed=32)
    w64 = stored(w)
    want = npl.forward(c, w64, tokens).to(torch.float32)

    def other(change):
        c2, w2 = json.loads(json.dumps(c)), dict(w64)
        change(c2, w2)
        return (npl.forward(c2, w2, tokens).float() - want).abs().max().item()
    assert other(lambda c2, w2: c2["layers"][0]["mixer"]["left"].update(bias_max=24)) > 0.05
    assert other(lambda c2, w2: w2.update({"l0.mix.left.sink": w64["l0.mix.left.sink"] - 40.0})) > 0.05
    assert other(lambda c2, w2: w2.update({"l0.mix.left.temp": torch.ones(4, dtype=torch.float64)})) > 0.05
    for sizes, tail, page in ((None, 0, 16), ((2,), 0, 4), ((7, 1, 30), 0, 8), (None, 60, 16)):
        steps, out = special(tmp_path, c, w, tokens, dtype, sizes=sizes, tail=tail, page=page)
        compare(steps, out, 70, {"r": want}, dtype, case="nufapel bias edges, sink, temperature")


def long_memory_model(kind, others):
    """One layer whose state forgets almost nothing (decays of nearly one and no removal for the delta rule, a forget
    gate of nearly one for the matrix memory, whose attention side is switched off by its output weight), without
    position vectors, in which the last token (2) reads what token 1 wrote wherever that stood.  Token 1's embedding
    is the first unit vector, token 2's the second, no other token has either component (and the norm's offset is
    zero, so that none gets one).  In every head the first column of the key matrix is a vector b to which the other
    columns, times `others`, are made orthogonal, and the second column of the query matrix is three times b: token
    1's key is b, every other key is orthogonal to it, and token 2's query reads along b only."""
    if kind == "delta":
        c = config(60, 32, [layer(delta(2, 16, rank=4), None)], eps=1e-6, softcap=40.0, max_positions=700)
        key, query, H, D = "l0.mix.k", "l0.mix.r", 2, 16
    else:
        c = config(60, 32, [layer(pair(2, 1, 16, 8, 2, 16, 8, bias_max=20, buckets=6, cap=12.0), None)], eps=1e-6,
                   softcap=40.0, max_positions=700)
        key, query, H, D = "l0.mix.right.k", "l0.mix.right.q", 2, 16
    w = make_weights(c, seed=33)
    w["pos"] *= 0.0
    w["embed"][:, :2] = 0.0
    w["embed"][1] = 0.0
    w["embed"][1, 0] = 4.0
    w["embed"][2] = 0.0
    w["embed"][2, 1] = 4.0
    w["l0.norm1.b"][:] = 0.0
    w["l0.norm1"][:2] = 1.0
    g = torch.Generator().manual_seed(34)
    wk = w[key].view(H, D, 32).clone()
    for blk in range(H):
        b = torch.randn(D, generator=g)
        b = b / b.norm()
        rest = wk[blk][:, 1:]
        wk[blk][:, 1:] = others * (rest - b[:, None] * (b @ rest)[None, :])
        wk[blk][:, 0] = b
    w[key] = wk.reshape(H * D, 32).contiguous()
    w[query][:, 1] = 3.0 * w[key][:, 0]
    if kind == "delta":
        w["l0.mix.w0"][:] = -14.0
        w["l0.mix.w2"] *= 0.0
        w["l0.mix.a.b"][:] = -14.0
        w["l0.mix.a"] *= 0.0
    else:
        w["l0.mix.right.f"] *= 0.0
        w["l0.mix.right.f.b"][:] = 11.5
        w["l0.mix.right.i"] *= 0.1
        w["l0.mix.left.out"] *= 0.0
    return c, w


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far", [0, 1, 63, 64, 300])
@pytest.mark.parametrize("kind", ["delta", "memory"])
def test_a_token_far_back_in_the_state(kind, far, dtype, tmp_path):
    """Token 1 stands at position `far` only among 500 tokens and the last token reads its trace in the state: taking it
    away changes the plain implementation's last logits greatly, and the engine's equal the plain ones whole, in
    portions and decoded (a state that is lost, restarted or overwritten at a portion's edge loses that token)."""
    c, w = long_memory_model(kind, 0.05)
    w64 = stored(w)
    tokens = [3 + (i * 7) % 11 for i in range(500)]
    tokens[far], tokens[-1] = 1, 2
    want = npl.forward(c, w64, tokens).to(torch.float32)
    without = list(tokens)
    without[far] = 4
    gone = npl.forward(c, w64, without).to(torch.float32)
    assert (want[-1] - gone[-1]).abs().max() > 0.3
    for sizes, tail in ((None, 0), ((100, 3, 2), 0), (None, 9)):
        steps, out = special(tmp_path, c, w, tokens, dtype, sizes=sizes, tail=tail)
        compare(steps, out, 60, {"r": want}, dtype, case=f"nufapel far token in the state ({kind})")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_tokens_of_a_memory_with_small_input_gates(dtype, tmp_path):
    """Input gates far below zero: the running maximum, which starts at 0 and not at the first gate, then decides the
    size of the first tokens' outputs (exp(i - m) is tiny, the denominator is exp(-m)); decoded from the second token
    on, and in portions of two."""
    c = config(64, 32, [layer(pair(2, 2, 8, 8, 2, 12, 20, bias_max=10, buckets=4, cap=9.0), dense(24))], eps=1e-6,
               loop=(0, 1, 2))
    w = make_weights(c, seed=35)
    w["l0.mix.right.i.b"][:] = -7.0
    w["l0.mix.right.f.b"][:] = 3.0
    tokens = random_tokens(24, 64, seed=36)
    want = npl.forward(c, stored(w), tokens).to(torch.float32)
    for sizes, tail in ((None, 0), ((2,), 0), (None, 23)):
        steps, out = special(tmp_path, c, w, tokens, dtype, sizes=sizes, page=4, tail=tail)
        compare(steps, out, 64, {"r": want}, dtype, case="nufapel first tokens of the memory")


# ----------------------------------------------------------- generation, scheduler, entry point
def plain_greedy(c, w, prompt, n):
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(npl.forward(c, w, seq)[-1].argmax()))
    return seq[len(prompt):]


def test_greedy_generation_through_the_entry_point(tmp_path):
    """make_driver + generate: the scheduler's portions, decode steps from captured graphs, sampling; 40 tokens each."""
    from jax_vllm_b200 import SamplingParams, generate, load_from_path, make_driver
    c = CONFIGS["na"]
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
    c = CONFIGS["nb"]
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
    assert d.stats.preemptions > 0
    w = stored(weights)
    for i, prompt in enumerate(prompts):
        assert d.requests[ids[i]].output_ids == plain_greedy(c, w, prompt, new_tokens[i]), f"request {i}"


def test_command_line(tmp_path):
    """cli.py as a user runs it on a Nufapel folder: prompts as token ids, 32-bit; the printed ids are the plain
    implementation's greedy tokens."""
    c = CONFIGS["nd"]
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


def random_configuration(seed):
    """A configuration drawn at random: every size, the order of the layers, the loop and the feed-forwards."""
    import random
    rng = random.Random(seed)
    width = rng.choice([24, 40, 56, 64])
    layers = []
    for _ in range(rng.randrange(1, 4)):
        if rng.random() < 0.5:
            mixer = delta(rng.randrange(1, 4), rng.choice([4, 12, 16, 20, 32]), rank=rng.randrange(1, 9))
        else:
            kv = rng.randrange(1, 3)
            mixer = pair(kv * rng.randrange(1, 4), kv, rng.choice([8, 16, 24, 32]), rng.choice([8, 16, 40]), rng.randrange(1, 3),
                         rng.choice([4, 10, 16, 32]), rng.choice([6, 16, 24]), scale=rng.uniform(0.1, 0.5),
                         bias_max=rng.randrange(5, 60), buckets=rng.choice([2, 4, 6, 9]), cap=rng.uniform(3.0, 20.0))
            mixer["mixer"]["left"]["bias_max"] = max(mixer["mixer"]["left"]["bias_max"], mixer["buckets"] // 2 + 1)
        kind = rng.random()
        if kind < 0.3:
            ff = None
        elif kind < 0.6:
            ff = dense(rng.randrange(8, 64))
        else:
            groups = rng.randrange(1, 4)
            per = rng.randrange(1, 4)
            keep = rng.randrange(1, groups + 1)
            ff = moe(groups * per, rng.randrange(1, keep * per + 1), groups, keep, rng.randrange(8, 40),
                     scale=rng.uniform(0.5, 2.5), limit=rng.uniform(1.0, 4.0))
        layers.append(layer(mixer, ff))
    loop = None
    if rng.random() < 0.6:
        a = rng.randrange(0, len(layers))
        loop = (a, rng.randrange(a + 1, len(layers) + 1), rng.randrange(1, 4))
    return config(rng.randrange(40, 200), width, layers, eps=10 ** rng.uniform(-6, -4), loop=loop,
                  softcap=rng.uniform(10.0, 60.0), max_positions=128)


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(seed, tmp_path):
    """Sizes, layer order, loop and options drawn at random; two requests as portions beside single tokens, 32-bit."""
    c = random_configuration(seed)
    weights = make_weights(c, seed=200 + seed)
    folder = write_folder(tmp_path / "model", c, weights)
    seqs = {"r0": random_tokens(50, c["vocab"], seed=300 + seed), "r1": random_tokens(31, c["vocab"], seed=400 + seed)}
    want = {rid: npl.forward(c, stored(weights), t).to(torch.float32) for rid, t in seqs.items()}
    plan = [{"r0": 13}, {"r0": 1, "r1": 9}, {"r0": 2, "r1": 1}, {"r0": 999, "r1": 1}, {"r1": 999}]
    fed, steps = {r: 0 for r in seqs}, []
    for k, row in enumerate(plan):
        entries = []
        for rid, n in row.items():
            part = seqs[rid][fed[rid]:fed[rid] + n]
            entries.append({"id": rid, "tokens": part, "want": list(range(len(part)))})
            fed[rid] += len(part)
        steps.append({"step": k, "entries": entries, "end": [e["id"] for e in entries if fed[e["id"]] == len(seqs[e["id"]])]})
    from jax_vllm_b200.engine.replay import Replayer
    rep = Replayer(folder, "float32", tmp_path / "out", max_tokens=128, page_size=8)
    rep.run_stream(json.dumps(s) for s in steps)
    compare(steps, tmp_path / "out", c["vocab"], want, "float32", case="nufapel random configurations")
