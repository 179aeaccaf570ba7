"""Decode and prefill throughput of the engine on one B200, for the Qwen3-8B shape with
random bfloat16 weights: the reference's headline metric (decoded tokens per second) at its largest
dense Qwen3 configuration.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]
    python bench.py --workload mixed14b|long32b      # a serving workload of a larger shape (its own JSON line)

Prints ONE JSON line.  `value` is decoded tokens per second at the given batch, each request
holding 2,048 tokens of context, timed on the device with CUDA events over K decode steps
after W warm-up steps (a "step" is one decode step: one token for every request of the
batch).  `e2e` is the same through the Python entry point (`add_request`/`step`), token ids
from the host and sampled tokens back to the host in every step.  `prefill` is one
2,048-token prompt in one step; `points` holds decoding at batch 1 and 64; `roofline` is
the decode step's bytes (every weight it uses once, and the cache of the live requests)
over its time, against the measured copy bandwidth.  Weights (15 GB) are far larger than
the L2, so nothing is flushed between iterations.  The engine runs on one GPU only: for
--gpus N > 1 it says so and exits with 2.
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], vocab_size=151936, hidden_size=4096, intermediate_size=12288,
                num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=40960, tie_word_embeddings=False)
CONTEXT = 2048
PREFILL_TOKENS = 2048
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"]))}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.proc = None
        self.index = index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.summary = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        mhz, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                mhz.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if mhz:
            self.summary = {"sm_mhz": statistics.median(mhz), "sm_max_mhz": max(mx), "reasons": sorted(reasons)}


def layer_params(c):
    H, I, D = c["hidden_size"], c["intermediate_size"], c["head_dim"]
    Hq, Hkv = c["num_attention_heads"], c["num_key_value_heads"]
    return H * (Hq + 2 * Hkv) * D + Hq * D * H + 3 * H * I


def decode_bytes(c, layers, batch, ctx, itemsize=2):
    weights = (layers * layer_params(c) + c["vocab_size"] * c["hidden_size"]) * itemsize
    kv = batch * ctx * layers * 2 * c["num_key_value_heads"] * c["head_dim"] * itemsize
    return weights + kv


def prefill_flops(c, layers, T):
    gemm = 2 * T * layers * layer_params(c) + 2 * c["vocab_size"] * c["hidden_size"]
    attn = layers * 4 * c["num_attention_heads"] * c["head_dim"] * T * (T + 1) // 2
    return gemm + attn


def fake_context(driver, batch, ctx):
    """`batch` live requests that hold `ctx` tokens each, their pages filled with random keys and values
    (what the tokens were does not change the work of a decode step)."""
    import torch
    rcs = []
    for i in range(batch):
        rc = driver.cache.admit(("bench", i))
        driver.cache.grow(rc, ctx)
        rc.num_tokens = ctx
        rcs.append(rc)
    for grp in driver.cache.groups:
        grp.k.normal_(0, 1)
        grp.v.normal_(0, 1)
    torch.cuda.synchronize()
    return rcs


MIN_TIMED_SECONDS = 0.5      # a timed region shorter than this is repeated until it adds up to it
MAX_CONTEXT = 4096            # requests of the decode runs never grow beyond this


def time_decode(model, batch, steps, warmup, ctx=CONTEXT):
    """Device time of `steps` decode steps at `batch`, repeated until MIN_TIMED_SECONDS are timed (at most until the
    requests reach MAX_CONTEXT tokens); returns (median ms per step over the repeats, launches per step, repeats,
    all the repeats' ms per step)."""
    import torch
    from jax_vllm_b200 import make_driver, ops
    from jax_vllm_b200.engine import StepEntry
    max_len = MAX_CONTEXT
    driver = make_driver(model, max_num_seqs=batch, max_model_len=max_len, block_size=PAGE, prefix_cache=False)
    rcs = fake_context(driver, batch, ctx)
    runner, cache, sampler = driver.runner, driver.cache, driver.sampler

    def one(i):
        entries = []
        for b, rc in enumerate(rcs):
            cache.grow(rc, rc.num_tokens + 1)
            entries.append(StepEntry(rc, [(i * 7919 + b) % 1000], (0,)))
        logits = runner.step(entries)
        toks = sampler.greedy(logits)
        for e in entries:
            rc = e.cache
            rc.num_tokens += 1
        return toks

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    per_step, launches, done = [], 0, warmup
    most = max(1, (MAX_CONTEXT - ctx - warmup - 1) // steps)
    while True:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        before = ops.launch_count
        start.record()
        for i in range(steps):
            one(done + i)
        end.record()
        torch.cuda.synchronize()
        done += steps
        per_step.append(start.elapsed_time(end) / steps)
        launches = (ops.launch_count - before) // steps
        if sum(per_step) * steps >= MIN_TIMED_SECONDS * 1e3 or len(per_step) >= most:
            break
    runner.check_kernels()
    del driver, runner, cache
    torch.cuda.empty_cache()
    return statistics.median(per_step), launches, len(per_step), per_step


def time_prefill(model, tokens, warmup, reps=3):
    import torch
    from jax_vllm_b200 import make_driver
    from jax_vllm_b200.engine import StepEntry
    max_len = -(-(tokens + 16) // PAGE) * PAGE
    driver = make_driver(model, max_num_seqs=1, max_model_len=max_len, block_size=PAGE, prefix_cache=False,
                         max_tokens_per_step=tokens)
    ids = [(i * 7919 + 13) % 1000 for i in range(tokens)]
    times = []
    for r in range(warmup + reps):
        rc = driver.cache.admit(("prefill", r))
        driver.cache.grow(rc, tokens)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        driver.runner.step([StepEntry(rc, ids, (tokens - 1,))])
        e.record()
        torch.cuda.synchronize()
        if r >= warmup:
            times.append(s.elapsed_time(e))
        driver.cache.release(("prefill", r))
    driver.runner.check_kernels()
    del driver
    torch.cuda.empty_cache()
    return statistics.median(times)


def time_e2e(model, batch, steps, warmup, ctx=CONTEXT):
    """Through the entry point: `batch` prompts of `ctx` tokens from the host, then decode steps whose
    sampled tokens come back to the host each step."""
    import torch
    from jax_vllm_b200 import SamplingParams, add_request, make_driver, step
    runs = max(3, min(25, int(MIN_TIMED_SECONDS / (steps * 0.004)) + 1))
    new = min(warmup + runs * steps + 4, MAX_CONTEXT - ctx)
    runs = max(1, (new - warmup - 4) // steps)
    max_len = -(-(ctx + new) // PAGE) * PAGE
    driver = make_driver(model, max_num_seqs=batch, max_model_len=max_len, block_size=PAGE, prefix_cache=False,
                         max_tokens_per_step=max(2048, batch))
    for b in range(batch):
        add_request(driver, [(i * 31 + b * 977) % 50000 for i in range(ctx)], SamplingParams(max_new_tokens=new))
    while any(len(r.output_ids) < 1 + warmup for r in driver.requests.values()):   # prompts, then warm-up decodes
        step(driver)
    # `runs` runs of `steps` steps (a run is tens of milliseconds of wall clock on a shared host, where one hiccup of
    # the host halves it): the median counts, the fastest is given beside it
    rates = []
    for _ in range(runs):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        emitted = 0
        for _ in range(steps):
            emitted += len(step(driver))
        torch.cuda.synchronize()
        rates.append(emitted / (time.perf_counter() - t0))
    # one copy per step: the batch description (tokens, positions, block tables, work lists) and, behind it in
    # the same buffer, seeds, counters and temperatures of the sampler
    g = driver.runner.graphs_sampled.get(batch)
    if g is not None:
        h2d = g.total * 4
    else:
        g = driver.runner.graphs.get(batch)
        h2d = (g.layout.total * 4 if g is not None else 0) + batch * (4 + 16)
    d2h = (batch + 1) * 4                        # sampled tokens and the kernels' status word
    del driver
    torch.cuda.empty_cache()
    return statistics.median(rates), max(rates), len(rates), h2d, d2h


def micro(spec: str, reps: int, eager: bool = False) -> int:
    """One kernel alone on data larger than the L2, for profiling:
    gemm:<N>x<K>:<M>:<impl>  the prompt product, impl = tcgen05 | tcgen05_swiglu | library (cuBLAS)
    linear:<N>x<K>:<M>[:parts][:stream|:skinny|:library]   the decode product of M rows with an [N, K] weight (several weights in turn):
                         as the engine picks it, or the tcgen05 kernel, the mma.sync kernel, cuBLAS
    attn_decode:<B>:<CTX>[:<SPLIT>[:<PAGE>[:<KV HEADS>[:<QUERY HEADS PER KV HEAD>]]]]   split decode attention of B requests with CTX cached tokens (8B head layout,
                         several caches in turn so that none stays in the L2), mma.sync kernel
    attn_decode_tcgen05:<B>:<CTX>[:<SPLIT>[:<PAGE>]]   the same with the tcgen05 kernel
    (the decode kernels are timed as replays of a CUDA graph of one launch per cache, as the engine runs them)
    attn_prefill:<T>     prompt attention of one request of T tokens (8B head layout), mma.sync kernel
    attn_prefill_tcgen05:<T>[:<PAGE>]   the same with the tcgen05 kernel
    attn_general:<T>:<HQ>:<HK>:<HV>:<KD>:<VD>[:<CAP>[:sigmoid]]   prompt attention of one request of T tokens with the mma.sync
                         kernel compiled for keys of KD and values of VD (HQ query, HK key, HV value heads)"""
    import torch
    from jax_vllm_b200 import ops
    kind, *rest = spec.split(":")
    dev = "cuda:0"
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if kind == "gemm":           # gemm:<N>x<K>:<M>:<impl>  impl = tcgen05 | tcgen05_swiglu | library
        n, k = (int(v) for v in rest[0].split("x"))
        m, impl = int(rest[1]), rest[2]
        copies = max(2, int(300e6 // (n * k * 2)) + 1)
        ws = [(torch.randn(n, k, device=dev) * 0.02).to(torch.bfloat16) for _ in range(copies)]
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        if impl == "library":
            run = lambda i: torch.mm(x, ws[i % copies].t())
        else:
            run = lambda i: ops.gemm_tcgen05(x, ws[i % copies], "swiglu" if impl.endswith("swiglu") else "bf16")
        for i in range(3):
            run(i)
        torch.cuda.synchronize()
        start.record()
        for i in range(reps):
            run(i)
        end.record()
        torch.cuda.synchronize()
        us = start.elapsed_time(end) / reps * 1e3
        print(json.dumps({"micro": spec, "us": round(us, 2), "TFLOP/s": round(2.0 * m * n * k / us / 1e6, 1)}))
        return 0
    if kind == "attn_general":
        T, hq, hk, hv, kd, vd = (int(v) for v in rest[:6])
        cap = float(rest[6]) if len(rest) > 6 else 0.0
        sigmoid = "sigmoid" in rest[7:]
        page = PAGE
        num_pages = -(-T // page)
        table = torch.randperm(num_pages).to(torch.int32).view(1, -1).to(dev)
        kc = torch.randn(num_pages, page, hk, kd, device=dev).to(torch.bfloat16)
        vc = torch.randn(num_pages, page, hv, vd, device=dev).to(torch.bfloat16)
        q = torch.randn(T, hq * kd, device=dev).to(torch.bfloat16)
        out = torch.empty(T, hq * vd, device=dev, dtype=torch.bfloat16)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        st = torch.zeros(1, dtype=torch.int32, device=dev)
        tpt = ops.attn_general_mma_tokens_per_tile(hq, hk)
        work = torch.tensor([[0, t] for t in range(0, T, tpt)], dtype=torch.int32, device=dev)
        bias = torch.zeros(hq, device=dev) if sigmoid else None
        run = lambda i: ops.attn_general_mma(q, hq * kd, out, kc, vc, table, cu, st, work, work.shape[0], hq, hk, kd ** -0.5,
                                             score_cap=cap, sigmoid=sigmoid, bias=bias)
        for i in range(3):
            run(i)
        torch.cuda.synchronize()
        start.record()
        for i in range(reps):
            run(i)
        end.record()
        torch.cuda.synchronize()
        ops.check_status()
        us = start.elapsed_time(end) / reps * 1e3
        flops = 2.0 * hq * (kd + vd) * T * (T + 1) / 2
        print(json.dumps({"micro": spec, "us": round(us, 2), "TFLOP/s": round(flops / us / 1e6, 1)}))
        return 0
    if kind == "linear":
        n, k = (int(v) for v in rest[0].split("x"))
        m = int(rest[1])
        copies = max(2, int(400e6 // (n * k * 2)) + 1)
        ws = [(torch.randn(n, k, device=dev) * 0.02).to(torch.bfloat16) for _ in range(copies)]
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        parts_ok = "parts" in rest[2:]        # let the kernel cut k and leave the parts of a sum
        if "skinny" in rest[2:]:              # the mma.sync kernel, whatever the dispatcher would take
            run = lambda i: ops.linear_skinny(x, ws[i % copies], torch.bfloat16, parts_ok)
        elif "stream" in rest[2:]:            # the tcgen05 product for larger batches, whatever the rows
            run = lambda i: ops.linear_stream(x, ws[i % copies], torch.bfloat16, parts_ok)
        elif "library" in rest[2:]:
            run = lambda i: torch.mm(x, ws[i % copies].t())
        else:
            run = lambda i: ops.linear(x, ws[i % copies], parts_ok=parts_ok)
        nbytes = n * k * 2
    else:
        hq, hkv, d, page = 32, 8, 128, PAGE
        if kind.startswith("attn_decode"):
            b, ctx = int(rest[0]), int(rest[1])
            split = int(rest[2]) if len(rest) > 2 else 256
            page = int(rest[3]) if len(rest) > 3 else PAGE
            if len(rest) > 4:
                hkv = int(rest[4]); hq = (int(rest[5]) if len(rest) > 5 else 4) * hkv
            q_lens = [1] * b
        else:
            b, ctx, q_lens = 1, 0, [int(rest[0])]
            page = int(rest[1]) if len(rest) > 1 else PAGE
        total = [ctx + q for q in q_lens]
        pages_per = [-(-t // page) for t in total]
        num_pages = sum(pages_per)
        table = torch.full((b, max(pages_per)), -1, dtype=torch.int32)
        perm = torch.randperm(num_pages).tolist()
        for e in range(b):
            for i in range(pages_per[e]):
                table[e, i] = perm.pop()
        copies = max(1, int(300e6 // (num_pages * page * hkv * d * 4))) + 1 if kind.startswith("attn_decode") else 1
        kcs = [torch.randn(num_pages, page, hkv, d, device=dev).to(torch.bfloat16) for _ in range(copies)]
        vcs = [torch.randn(num_pages, page, hkv, d, device=dev).to(torch.bfloat16) for _ in range(copies)]
        kc, vc = kcs[0], vcs[0]
        n_tok = sum(q_lens)
        q = torch.randn(n_tok, hq * d, device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)
        cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=dev)
        st = torch.tensor([ctx] * b, dtype=torch.int32, device=dev)
        common = (kc, vc, table.to(dev), cu, st)
        if kind.startswith("attn_decode"):
            work = torch.tensor([[e, 0] for e in range(b)], dtype=torch.int32, device=dev)
            n_splits = -(-max(total) // split)
            if kind == "attn_decode_tcgen05":
                run = lambda i: ops.attn_decode_tcgen05(q, hq * d, out, kcs[i % copies], vcs[i % copies], *common[2:], work,
                                                        b, hq, hkv, d, d ** -0.5)
            else:
                run = lambda i: ops.attn_mma(q, hq * d, out, kcs[i % copies], vcs[i % copies], *common[2:], work, b, hq,
                                             hkv, d, 0, d ** -0.5, split_size=split, n_splits=n_splits)
        elif kind == "attn_prefill_tcgen05":
            tpt = ops.attn_tcgen05_tokens_per_tile(hq, hkv)
            work = torch.tensor([[0, t] for t in range(0, q_lens[0], tpt)], dtype=torch.int32, device=dev)
            run = lambda i: ops.attn_tcgen05(q, hq * d, out, *common, work, work.shape[0], hq, hkv, d, d ** -0.5)
        else:
            tpt = ops.attn_mma_tokens_per_tile(hq, hkv)
            work = torch.tensor([[0, t] for t in range(0, q_lens[0], tpt)], dtype=torch.int32, device=dev)
            run = lambda i: ops.attn_mma(q, hq * d, out, *common, work, work.shape[0], hq, hkv, d, 0, d ** -0.5)
        nbytes = 2 * kc.numel() * 2
    for i in range(3):
        run(i)
    torch.cuda.synchronize()
    if (kind.startswith("attn_decode") or kind == "linear") and not eager:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(copies):
                run(i)
        graph.replay()
        torch.cuda.synchronize()
        start.record()
        for i in range(reps):
            graph.replay()
        end.record()
        reps *= copies
    else:
        start.record()
        for i in range(reps):
            run(i)
        end.record()
    torch.cuda.synchronize()
    ops.check_status()
    us = start.elapsed_time(end) / reps * 1e3
    print(json.dumps({"micro": spec, "us": round(us, 2), "GB/s": round(nbytes / us / 1e3, 1)}))
    return 0


def timeline(batch: int, layers: int, shape=None) -> int:
    """Start, duration and end of every kernel of one replayed decode step (torch's profiler; programmatic dependent
    launch lets kernels overlap, so a kernel's start is when its first block became resident, and the increments from
    end to end tell what each adds to the step): `python bench.py --timeline 8 --layers 4`; with `--workload NAME`
    the layer sizes of that workload's shape instead of the 8B ones."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    from jax_vllm_b200 import make_driver, random_model, registry
    from jax_vllm_b200.engine import StepEntry
    cfg = dict(QWEN3_8B, **(WORKLOADS[shape]["config"] if shape else {}))
    model = random_model(registry.config_from_dict(dict(cfg, num_hidden_layers=layers)), seed=5, dtype="bf16")
    driver = make_driver(model, max_num_seqs=batch, max_model_len=CONTEXT + 64, block_size=PAGE, prefix_cache=False)
    rcs = fake_context(driver, batch, CONTEXT)

    def one(i):
        entries = []
        for b, rc in enumerate(rcs):
            driver.cache.grow(rc, rc.num_tokens + 1)
            entries.append(StepEntry(rc, [(i * 7919 + b) % 1000], (0,)))
        driver.runner.step(entries)
        for rc in rcs:
            rc.num_tokens += 1

    for i in range(6):
        one(i)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        one(7)
        torch.cuda.synchronize()
    evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA), key=lambda e: e.time_range.start)
    t0, last_end = evs[0].time_range.start, evs[0].time_range.start
    print(f"decode step, batch {batch}, {CONTEXT}-token context, {layers} layers: start, duration, end, end minus the latest end before (us)")
    for e in evs:
        start, dur = e.time_range.start - t0, e.time_range.end - e.time_range.start
        print(f"{start:9.1f} {dur:7.1f} {start + dur:9.1f} {e.time_range.end - last_end:+7.1f}  {e.name[:70]}")
        last_end = max(last_end, e.time_range.end)
    return 0


WORKLOADS = {
    # the larger dense Qwen3 shapes as serving workloads: all requests arrive at once, the scheduler cuts their
    # prompts into portions beside the decode tokens of the others
    "mixed14b": dict(config=dict(hidden_size=5120, intermediate_size=17408, num_hidden_layers=40, num_attention_heads=40),
                     seed=6, requests=32, prompt=(128, 4096), prompt_seed=7, shared_prefix=1024, new_tokens=256,
                     tokens_per_step=512),
    "long32b": dict(config=dict(hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64),
                    seed=8, requests=16, prompt=(8192, 8192), prompt_seed=9, shared_prefix=0, new_tokens=512,
                    tokens_per_step=2048),
}


def workload(name: str, layers) -> int:
    """Runs one of WORKLOADS through the entry point and prints one JSON line: wall-clock seconds, prompt and
    generated tokens per second, time to the first token, and the steps by kind (with a portion of a prompt
    in them, or decoding alone) with their time and the tokens they ran."""
    import random
    import torch
    from jax_vllm_b200 import SamplingParams, add_request, has_work, make_driver, prewarm, random_model, registry, step
    w = WORKLOADS[name]
    cfg_dict = dict(QWEN3_8B, **w["config"])
    if layers:
        cfg_dict["num_hidden_layers"] = layers
    model = random_model(registry.config_from_dict(cfg_dict), seed=w["seed"], dtype="bf16", device="cuda:0")
    rng = random.Random(w["prompt_seed"])
    vocab = cfg_dict["vocab_size"]
    shared = [rng.randrange(vocab) for _ in range(w["shared_prefix"])]
    prompts = []
    for i in range(w["requests"]):
        n = rng.randint(*w["prompt"])
        own = [rng.randrange(vocab) for _ in range(n)]
        prompts.append((shared + own[len(shared):]) if shared and i % 2 == 0 and n > len(shared) else own)
    longest = max(len(p) for p in prompts)
    max_len = -(-(longest + w["new_tokens"]) // PAGE) * PAGE
    driver = make_driver(model, max_num_seqs=w["requests"], max_model_len=max_len, max_prefill_len=longest,
                         block_size=PAGE, max_tokens_per_step=w["tokens_per_step"])
    warm = prewarm(driver)
    torch.cuda.synchronize()
    st = driver.stats
    kinds = {"with_prompt": [0, 0.0, 0], "decode_only": [0, 0.0, 0]}          # steps, seconds, tokens run
    with ClockSampler() as clocks:
        t0 = time.perf_counter()
        ids = [add_request(driver, p, SamplingParams(max_new_tokens=w["new_tokens"])) for p in prompts]
        reqs = [driver.requests[i] for i in ids]
        while has_work(driver):
            t1 = time.perf_counter()
            before = (st.prefill_tokens, st.decode_tokens)
            step(driver)
            rec = kinds["with_prompt" if st.prefill_tokens > before[0] else "decode_only"]
            rec[0] += 1
            rec[1] += time.perf_counter() - t1
            rec[2] += st.prefill_tokens + st.decode_tokens - sum(before)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    n_prompt, n_new = sum(len(p) for p in prompts), sum(len(r.output_ids) for r in reqs)
    ttft = sorted(r.first_token_time - r.arrival for r in reqs)
    out = {"workload": name, "layers": cfg_dict["num_hidden_layers"], "requests": len(prompts), "prompt_tokens": n_prompt,
           "new_tokens": n_new, "seconds": round(dt, 3), "tokens_per_s": round((n_prompt + n_new) / dt, 1),
           "new_tokens_per_s": round(n_new / dt, 1),
           "ttft_s": {"median": round(ttft[len(ttft) // 2], 3), "max": round(ttft[-1], 3)}, "steps": st.steps}
    for kind, (n, sec, toks) in kinds.items():
        out["steps_" + kind] = {"steps": n, "ms_per_step": round(1e3 * sec / max(1, n), 2),
                                "tokens_per_s": round(toks / max(1e-9, sec), 1)}
    out.update({"preemptions": st.preemptions, "prefix_hit_tokens": st.cache_hit_tokens, "prewarm_s": round(warm, 1),
                "gb_allocated": round(torch.cuda.max_memory_allocated() / 1e9, 1),
                "clocks": clocks.summary})
    print(json.dumps(out))
    return 0


# ------------------------------------------------------------------ the Guronex design beside Qwen3
# Layer sizes for `--design guronex`: each a Guronex layer (latent attention + routed experts + token input) and the
# Qwen3 dense layer of equal width, equal number of heads and about equal feed-forward work per token
# (3 * intermediate = 2 * top * expert size).  "lite": the width, experts and expert size of a 16B-class mixture
# with a cache row of 128 (latent 64 + rotated 64), the size the tcgen05 attention kernels take; "mid": a wider
# one; "row576": the cache row of published latent-attention models (latent 512 + rotated 64), which runs on the
# CUDA-core attention kernel here.
DESIGN_SIZES = {
    "lite": dict(width=2048, heads=16, dim=64, rot=64, vdim=64, rank=64, experts=64, top=6, ff=1408, groups=(8, 4), side=64),
    "mid": dict(width=4096, heads=32, dim=96, rot=48, vdim=128, rank=80, experts=32, top=4, ff=2048, groups=(4, 2), side=64),
    "row576": dict(width=2048, heads=16, dim=128, rot=64, vdim=128, rank=512, experts=64, top=6, ff=1408, groups=(8, 4), side=64),
}


def design_configs(z, layers, vocab=32000):
    mixer = {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot"], "vdim": z["vdim"], "kv_rank": z["rank"],
             "rot": {"base": 10000.0, "dims": z["rot"]}, "scale": (z["dim"] + z["rot"]) ** -0.5}
    mlp = {"kind": "moe", "expert": {"ff": z["ff"]},
           "router": {"experts": z["experts"], "top": z["top"], "groups": {"count": z["groups"][0], "keep": z["groups"][1]}}}
    guronex = {"architecture": "Guronex", "vocab": vocab, "width": z["width"], "norm": {"eps": 1e-5}, "residual_mult": 0.5,
               "token_side": {"dim": z["side"]},
               "layers": [{"type": "latent_attention", "mixer": dict(mixer), "mlp": mlp} for _ in range(layers)]}
    inter = -(-(2 * z["top"] * z["ff"] // 3) // 128) * 128
    qwen = dict(QWEN3_8B, vocab_size=vocab, hidden_size=z["width"], intermediate_size=inter, num_hidden_layers=layers,
                num_attention_heads=z["heads"], num_key_value_heads=max(1, z["heads"] // 4), head_dim=128)
    return guronex, qwen


# Layer sizes for `--design loselix`: three layers, one of each of its mixers (softmax attention with a gate a head;
# sigmoid attention over normed projections; two capped score maps on shared values), each with a relu-squared
# feed-forward of `ff`, beside the Qwen3 dense layer of equal width, heads and feed-forward work per token
# (3 * intermediate = 2 * ff).  "w2k" and "w4k": heads of 128 throughout (two maps of 64 on values of 128), the sizes
# of 1B- and 8B-class models; "mix": heads of 64, 96 and 48/96, which run on the mma.sync kernels.
LOSELIX_SIZES = {
    "w2k": dict(width=2048, heads=16, kv=4, ff=8448, soft=(128, 128, 64), sig=128, twin=(64, 128, 32)),
    "w4k": dict(width=4096, heads=32, kv=8, ff=18432, soft=(128, 128, 64), sig=128, twin=(64, 128, 32)),
    "mix": dict(width=2048, heads=16, kv=4, ff=8448, soft=(64, 64, 32), sig=96, twin=(48, 96, 12)),
}
LOSELIX_KINDS = ("soft", "sigmoid", "twin")


def loselix_configs(z, layers, vocab=32000):
    H, G = z["heads"], z["kv"]
    sd, sv, sr = z["soft"]
    td, tv, tr = z["twin"]
    mlp = {"kind": "dense", "ff": z["ff"]}
    three = [{"type": "attention_2", "mlp": dict(mlp),
              "mixer": {"heads": H, "kv_heads": G, "dim": sd, "vdim": sv, "scale": sd ** -0.5, "rot": {"base": 5e5, "dims": sr}}},
             {"type": "attention_3", "mlp": dict(mlp),
              "mixer": {"heads": H, "kv_heads": G, "dim": z["sig"], "vdim": z["sig"], "scale": z["sig"] ** -0.5,
                        "q_temp": {"coef": 0.3, "every": 128}}},
             {"type": "attention", "mlp": dict(mlp),
              "mixer": {"heads": H, "kv_heads": G, "dim": td, "vdim": tv, "scale": td ** -0.5, "softcap": 50.0, "diff": 0.3,
                        "rot": {"base": 2.5e5, "dims": tr}}}]
    loselix = {"architecture": "Loselix", "vocab": vocab, "width": z["width"], "norm": {"eps": 1e-6},
               "layers": [dict(three[i % 3]) for i in range(layers)]}
    inter = -(-(2 * z["ff"] // 3) // 128) * 128
    qwen = dict(QWEN3_8B, vocab_size=vocab, hidden_size=z["width"], intermediate_size=inter, num_hidden_layers=layers,
                num_attention_heads=H, num_key_value_heads=G, head_dim=128)
    return loselix, qwen


def time_part(fn, reps, flush):
    """Median device time (us) of `fn`, captured into a CUDA graph (so that the host's launches do not count) and
    replayed one at a time, the L2 written over in between."""
    import torch
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    times = []
    for _ in range(reps):
        flush.add_(1)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); graph.replay(); e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e) * 1e3)
    return statistics.median(times)


def design_parts(model, kind, z, inter, batch, tokens, reps, pk, layer_index=0):
    """The attention kernel alone, the whole mixer and the whole feed-forward of layer 0: one prompt of `tokens`
    tokens, then one decode step of `batch` requests at CONTEXT tokens; each with its roofline (the slower of its
    FLOPs at the measured bf16 peak and its bytes, weights and cache rows read once, at the measured copy bandwidth)."""
    import torch
    from jax_vllm_b200 import make_driver
    from jax_vllm_b200.engine import StepEntry
    W, H = z["width"], z["heads"]
    flush = torch.zeros(160 << 20, dtype=torch.int16, device="cuda")
    out = {}
    layer = model.layers[layer_index]
    for phase in ("prefill", "decode"):
        if phase == "prefill":
            driver = make_driver(model, max_num_seqs=1, max_model_len=tokens + 16, block_size=PAGE, prefix_cache=False,
                                 max_tokens_per_step=tokens, cuda_graphs=False)
            rc = driver.cache.admit("p")
            driver.cache.grow(rc, tokens)
            entries = [StepEntry(rc, [(i * 7919 + 13) % 1000 for i in range(tokens)], (tokens - 1,))]
            n, pairs = tokens, tokens * (tokens + 1) // 2
        else:
            driver = make_driver(model, max_num_seqs=batch, max_model_len=CONTEXT + 64, block_size=PAGE, prefix_cache=False,
                                 cuda_graphs=False)
            rcs = fake_context(driver, batch, CONTEXT)
            for rc in rcs:
                driver.cache.grow(rc, rc.num_tokens + 1)
            entries = [StepEntry(rc, [b], (0,)) for b, rc in enumerate(rcs)]
            n, pairs = batch, batch * (CONTEXT + 1)
        step = driver.runner.builder.build(entries)
        cache = driver.runner.layer_caches[layer_index]
        table = step.block_tables[cache.group]
        x = (torch.randn((n, W), device="cuda") * 0.5).to(torch.bfloat16)
        mixer, ff = layer.mixer, layer.feed_forward
        if kind == "guronex":
            dk, dc = z["rank"] + z["rot"], z["rank"]
            q = torch.randn((n, H * dk), device="cuda").to(torch.bfloat16)
            attn = lambda: mixer.attend(q, step, cache, table)
            keys = tokens if phase == "prefill" else batch * (CONTEXT + 1)          # cache rows read, each once
            attn_flops, attn_bytes = 2 * H * (dk + dc) * pairs, keys * dk * 2 + n * H * (dk + dc) * 2
            hit = z["experts"] * (1 - (1 - z["top"] / z["experts"]) ** n)           # experts that some token chose, about
            ff_flops, ff_bytes = 2 * n * z["top"] * 2 * z["ff"] * W, hit * 2 * z["ff"] * W * 2
        elif kind == "loselix":
            hq, hk, hv, dk, dv = mixer.hq, mixer.hk, mixer.hv, mixer.d, mixer.dv     # as the kernels see them
            q = torch.randn((n, hq * dk), device="cuda").to(torch.bfloat16)
            a = torch.empty((n, hq * dv), dtype=torch.float32 if mixer.maps == 2 else torch.bfloat16, device="cuda")
            attn = lambda: mixer.attend(q, a, step, cache, table)
            keys = tokens if phase == "prefill" else batch * (CONTEXT + 1)
            attn_flops = 2 * hq * (dk + dv) * pairs
            attn_bytes = keys * (hk * dk + hv * dv) * 2 + n * hq * (dk * 2 + dv * a.element_size())
            ff_flops, ff_bytes = 2 * n * 2 * z["ff"] * W, 2 * z["ff"] * W * 2
        else:
            hkv = mixer.hkv
            qkv = torch.randn((n, (H + 2 * hkv) * 128), device="cuda").to(torch.bfloat16)
            o = torch.empty((n, H * 128), dtype=torch.bfloat16, device="cuda")
            attn = lambda: mixer.attend(qkv, o, step, cache, table)
            keys = tokens if phase == "prefill" else batch * (CONTEXT + 1)
            attn_flops, attn_bytes = 4 * H * 128 * pairs, keys * 2 * hkv * 128 * 2 + n * H * 128 * 2 * 2
            ff_flops, ff_bytes = 2 * n * 3 * inter * W, 3 * inter * W * 2
        res = {}
        for name, fn, flops, nbytes in (("attention kernel", attn, attn_flops, attn_bytes),
                                        ("mixer", lambda: mixer.forward(x, step, cache), None, None),
                                        ("feed-forward", lambda: ff.forward(x, step), ff_flops, ff_bytes)):
            us = time_part(fn, reps, flush)
            res[name] = {"us": round(us, 1)}
            if flops is not None:
                # the slower of the arithmetic at the measured bf16 peak and the bytes at the measured copy bandwidth
                t_flops, t_bytes = flops / (pk["bf16_tflops"] * 1e12) * 1e6, nbytes / (pk["hbm_gbs"] * 1e9) * 1e6
                ideal = max(t_flops, t_bytes)
                res[name].update(roofline_us=round(ideal, 1), bound="flops" if t_flops >= t_bytes else "bytes",
                                 of_roofline=round(ideal / us, 3))
        driver.runner.check_kernels()
        out[phase] = res
        del driver
        torch.cuda.empty_cache()
    return out


def design(name: str, layers, sizes, steps, warmup) -> int:
    """`--design guronex|loselix`: prefill and decode throughput of that design at a few layer sizes beside the Qwen3
    dense model of equal size (random weights, `--layers` layers, default 4; 3 for loselix, one of each mixer), and
    the attention kernel, the mixer and the feed-forward of one layer (for loselix: of each kind of layer) each alone
    with their rooflines."""
    import torch
    from jax_vllm_b200 import random_model, registry
    if name == "loselix":
        return design_loselix(layers or 3, sizes, steps, warmup)
    if name == "nufapel":
        return design_nufapel(layers or 3, sizes, steps, warmup)
    if name == "gogivik":
        return design_gogivik(layers or 3, sizes, steps, warmup)
    if name != "guronex":
        print(f"bench.py: no design {name!r}")
        return 2
    layers = layers or 4
    pk, pk_src = peaks()
    out = {"design": name, "layers": layers, "prefill_tokens": PREFILL_TOKENS, "decode_batch": 8, "context": CONTEXT,
           "dtype": "bf16", "data": "synthetic (random weights, seed 5)", "peaks": pk, "peak_source": pk_src, "sizes": {}}
    for tag in sizes:
        z = DESIGN_SIZES[tag]
        g_cfg, q_cfg = design_configs(z, layers)
        row = {"guronex": {"config": {k: v for k, v in z.items()}}, "qwen3": {"config": {
            "hidden": z["width"], "heads": z["heads"], "kv_heads": q_cfg["num_key_value_heads"], "head_dim": 128,
            "intermediate": q_cfg["intermediate_size"]}}}
        for kind, cfg in (("guronex", g_cfg), ("qwen3", q_cfg)):
            model = random_model(registry.config_from_dict(cfg), seed=5, dtype="bf16", device="cuda:0")
            with ClockSampler() as clocks:
                pms = time_prefill(model, PREFILL_TOKENS, warmup=2, reps=5)
                dms, launches, _, _ = time_decode(model, 8, steps, warmup)
            row[kind].update(prefill_tok_s=round(PREFILL_TOKENS / (pms / 1e3), 1), prefill_ms=round(pms, 3),
                             decode_tok_s=round(8 / (dms / 1e3), 1), decode_ms_per_step=round(dms, 4),
                             decode_launches_per_step=launches, clocks=clocks.summary)
            row[kind]["parts"] = design_parts(model, kind, z, q_cfg["intermediate_size"], 8, PREFILL_TOKENS, 7, pk)
            del model
            torch.cuda.empty_cache()
        out["sizes"][tag] = row
    print(json.dumps(out))
    return 0


def design_loselix(layers, sizes, steps, warmup) -> int:
    import torch
    from jax_vllm_b200 import random_model, registry
    pk, pk_src = peaks()
    sizes = [t for t in sizes if t in LOSELIX_SIZES] or list(LOSELIX_SIZES)
    out = {"design": "loselix", "layers": layers, "prefill_tokens": PREFILL_TOKENS, "decode_batch": 8, "context": CONTEXT,
           "dtype": "bf16", "data": "synthetic (random weights, seed 5)", "peaks": pk, "peak_source": pk_src, "sizes": {}}
    for tag in sizes:
        z = LOSELIX_SIZES[tag]
        l_cfg, q_cfg = loselix_configs(z, layers)
        row = {"loselix": {"config": dict(z)}, "qwen3": {"config": {
            "hidden": z["width"], "heads": z["heads"], "kv_heads": z["kv"], "head_dim": 128,
            "intermediate": q_cfg["intermediate_size"]}}}
        for kind, cfg in (("loselix", l_cfg), ("qwen3", q_cfg)):
            model = random_model(registry.config_from_dict(cfg), seed=5, dtype="bf16", device="cuda:0")
            with ClockSampler() as clocks:
                pms = time_prefill(model, PREFILL_TOKENS, warmup=2, reps=5)
                dms, launches, _, _ = time_decode(model, 8, steps, warmup)
            row[kind].update(prefill_tok_s=round(PREFILL_TOKENS / (pms / 1e3), 1), prefill_ms=round(pms, 3),
                             decode_tok_s=round(8 / (dms / 1e3), 1), decode_ms_per_step=round(dms, 4),
                             decode_launches_per_step=launches, clocks=clocks.summary)
            if kind == "qwen3":
                row[kind]["parts"] = design_parts(model, kind, z, q_cfg["intermediate_size"], 8, PREFILL_TOKENS, 7, pk)
            else:
                row[kind]["parts"] = {LOSELIX_KINDS[i]: design_parts(model, kind, z, 0, 8, PREFILL_TOKENS, 7, pk, layer_index=i)
                                      for i in range(min(3, layers))}
            del model
            torch.cuda.empty_cache()
        out["sizes"][tag] = row
    print(json.dumps(out))
    return 0


# ------------------------------------------------------------------ the Nufapel design beside Loselix
# Layer sizes for `--design nufapel`: three layers (attention with a distance bias and a sink beside a matrix memory,
# over a dense feed-forward; a delta-rule layer over routed experts; the pair again over routed experts), beside three
# Loselix softmax-attention layers of equal width, heads and feed-forward work per token.  "w2k": the width of a
# 1B-class model, a memory of 8 heads of 128 x 256 and delta heads of 64; "w4k": an 8B-class width, a memory of 8 heads
# of 256 x 512 (the sizes of a published 7B matrix-memory model) and delta heads of 64; "small": heads of 64 everywhere.
NUFAPEL_SIZES = {
    "w2k": dict(width=2048, heads=16, kv=4, dim=128, vdim=128, mem=(8, 128, 256), delta=(32, 64), rank=64, buckets=32,
                bias_max=1024, ff=8192, experts=32, top=4, eff=1024, groups=(4, 2)),
    "w4k": dict(width=4096, heads=32, kv=8, dim=128, vdim=128, mem=(8, 256, 512), delta=(64, 64), rank=96, buckets=32,
                bias_max=1024, ff=16384, experts=32, top=4, eff=2048, groups=(4, 2)),
    "small": dict(width=1024, heads=16, kv=4, dim=64, vdim=64, mem=(4, 64, 128), delta=(16, 64), rank=32, buckets=16,
                  bias_max=256, ff=4096, experts=16, top=2, eff=1024, groups=(2, 1)),
}
NUFAPEL_KINDS = ("pair_dense", "delta_moe", "pair_moe")
FP32_LANES = 148 * 128        # 32-bit multiply-adds a clock: 148 SMs of 128 lanes


def nufapel_configs(z, layers, vocab=32000):
    H, G = z["heads"], z["kv"]
    mh, md, mv = z["mem"]
    dh, dd = z["delta"]
    pair = {"left": {"heads": H, "kv_heads": G, "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
                     "bias_max": z["bias_max"], "buckets": z["buckets"]},
            "right": {"heads": mh, "dim": md, "vdim": mv, "gate_cap": 15.0}}
    dense = {"kind": "dense", "ff": z["ff"]}
    moe = {"kind": "moe", "expert": {"ff": z["eff"], "limit": 7.0},
           "router": {"experts": z["experts"], "top": z["top"], "scale": 1.0,
                      "groups": {"count": z["groups"][0], "keep": z["groups"][1]}}}
    three = [{"type": "parallel", "mixer": pair, "mlp": dense},
             {"type": "general_delta", "mixer": {"heads": dh, "dim": dd, "decay_rank": z["rank"]}, "mlp": moe},
             {"type": "parallel", "mixer": pair, "mlp": moe}]
    nufapel = {"architecture": "Nufapel", "vocab": vocab, "width": z["width"], "norm": {"eps": 1e-5},
               "max_positions": MAX_CONTEXT + 64, "logit_softcap": 30.0,
               "layers": [json.loads(json.dumps(three[i % 3])) for i in range(layers)]}
    soft = {"type": "attention_2", "mlp": {"kind": "dense", "ff": z["ff"]},
            "mixer": {"heads": H, "kv_heads": G, "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
                      "rot": {"base": 5e5, "dims": z["dim"] // 2}}}
    loselix = {"architecture": "Loselix", "vocab": vocab, "width": z["width"], "norm": {"eps": 1e-6},
               "layers": [json.loads(json.dumps(soft)) for _ in range(layers)]}
    return nufapel, loselix


def nufapel_parts(model, z, layer_index, batch, tokens, reps, pk, sm_mhz):
    """Layer `layer_index` of a Nufapel model in parts, each alone: the attention kernel, each recurrence (from the
    projected row to the heads before the output product: prepare, scan, norm and gate), the whole mixer, the whole
    feed-forward.  One prompt of `tokens` tokens, then one decode step of `batch` requests at CONTEXT tokens.
    Rooflines: attention and feed-forward as for the other designs (the slower of FLOPs at the measured bf16 peak and
    bytes at the measured copy bandwidth); a recurrence is 32-bit arithmetic on the CUDA cores by the design's rule
    (the state and all that enters it are 32-bit), so its roofline is the slower of its multiply-adds at 148 x 128
    lanes x the SM clock and its bytes (the state read and written once, the per-token vectors once)."""
    import torch
    from jax_vllm_b200 import make_driver
    from jax_vllm_b200.engine import StepEntry
    W = z["width"]
    flush = torch.zeros(160 << 20, dtype=torch.int16, device="cuda")
    layer = model.layers[layer_index]
    mixer, ff = layer.mixer, layer.feed_forward
    out = {}
    for phase in ("prefill", "decode"):
        if phase == "prefill":
            driver = make_driver(model, max_num_seqs=1, max_model_len=tokens + 16, block_size=PAGE, prefix_cache=False,
                                 max_tokens_per_step=tokens, cuda_graphs=False)
            rc = driver.cache.admit("p")
            driver.cache.grow(rc, tokens)
            entries = [StepEntry(rc, [(i * 7919 + 13) % 1000 for i in range(tokens)], (tokens - 1,))]
            n, pairs, keys, seqs = tokens, tokens * (tokens + 1) // 2, tokens, 1
        else:
            driver = make_driver(model, max_num_seqs=batch, max_model_len=CONTEXT + 64, block_size=PAGE, prefix_cache=False,
                                 cuda_graphs=False)
            rcs = fake_context(driver, batch, CONTEXT)
            for rc in rcs:
                driver.cache.grow(rc, rc.num_tokens + 1)
            entries = [StepEntry(rc, [b], (0,)) for b, rc in enumerate(rcs)]
            n, pairs, keys, seqs = batch, batch * (CONTEXT + 1), batch * (CONTEXT + 1), batch
        step = driver.runner.builder.build(entries)
        cache = driver.runner.layer_caches[layer_index]
        x = (torch.randn((n, W), device="cuda") * 0.5).to(torch.bfloat16)
        jobs = []

        def recurrence(part, view, removal):
            row = (torch.randn((n, part.in_rows), device="cuda") * 0.5).to(torch.bfloat16)
            heads = torch.empty((n, part.heads_out), dtype=torch.bfloat16, device="cuda")
            d = part.d
            v = part.heads_out // part.h
            fma = n * part.h * d * v * (4 if removal else 3)                  # decay, write, read (and remove: +1 dot, +1 update)
            nbytes = seqs * 2 * part.h * d * v * 4 + n * part.in_rows * 2 + n * part.heads_out * 2
            t_fma, t_bytes = fma / (FP32_LANES * sm_mhz * 1e6) * 1e6, nbytes / (pk["hbm_gbs"] * 1e9) * 1e6
            return (lambda: part.from_projection(row, step, view, heads)), (t_fma, t_bytes, "fp32 lanes")

        if hasattr(mixer, "sides"):
            att, mem = mixer.sides
            q = torch.randn((n, att.hq * att.d), device="cuda").to(torch.bfloat16)
            a = torch.empty((n, att.hq * att.dv), dtype=torch.bfloat16, device="cuda")
            table = step.block_tables[cache[0].group]
            flops = 2 * att.hq * (att.d + att.dv) * pairs
            nbytes = keys * (att.hk * att.d + att.hv * att.dv) * 2 + n * att.hq * (att.d + att.dv) * 2
            jobs.append(("attention kernel", lambda: att.attend(q, a, step, cache[0], table),
                         (flops / (pk["bf16_tflops"] * 1e12) * 1e6, nbytes / (pk["hbm_gbs"] * 1e9) * 1e6, "flops")))
            jobs.append(("memory recurrence",) + recurrence(mem, cache[1], False))
        else:
            jobs.append(("delta recurrence",) + recurrence(mixer, cache, True))
        jobs.append(("mixer", lambda: mixer.forward(x, step, cache), None))
        if ff is not None:
            if layer_index % 3 != 0:                                          # routed experts
                hit = z["experts"] * (1 - (1 - z["top"] / z["experts"]) ** n)
                ff_flops, ff_bytes = 2 * n * z["top"] * 3 * z["eff"] * W, hit * 3 * z["eff"] * W * 2
            else:
                ff_flops, ff_bytes = 2 * n * 2 * z["ff"] * W, 2 * z["ff"] * W * 2
            jobs.append(("feed-forward", lambda: ff.forward(x, step),
                         (ff_flops / (pk["bf16_tflops"] * 1e12) * 1e6, ff_bytes / (pk["hbm_gbs"] * 1e9) * 1e6, "flops")))
        res = {}
        for name, fn, roof in jobs:
            us = time_part(fn, reps, flush)
            res[name] = {"us": round(us, 1)}
            if roof is not None:
                t_math, t_bytes, unit = roof
                ideal = max(t_math, t_bytes)
                res[name].update(roofline_us=round(ideal, 1), bound=unit if t_math >= t_bytes else "bytes",
                                 of_roofline=round(ideal / us, 3))
        driver.runner.check_kernels()
        out[phase] = res
        del driver
        torch.cuda.empty_cache()
    return out


def design_nufapel(layers, sizes, steps, warmup) -> int:
    import torch
    from jax_vllm_b200 import random_model, registry
    pk, pk_src = peaks()
    sizes = [t for t in sizes if t in NUFAPEL_SIZES] or ["w2k", "w4k"]
    out = {"design": "nufapel", "layers": layers, "prefill_tokens": PREFILL_TOKENS, "decode_batch": 8, "context": CONTEXT,
           "dtype": "bf16", "data": "synthetic (random weights, seed 5)", "peaks": pk, "peak_source": pk_src, "sizes": {}}
    for tag in sizes:
        z = NUFAPEL_SIZES[tag]
        n_cfg, l_cfg = nufapel_configs(z, layers)
        row = {"nufapel": {"config": {k: v for k, v in z.items()}},
               "loselix": {"config": {"width": z["width"], "heads": z["heads"], "kv": z["kv"], "dim": z["dim"], "ff": z["ff"]}}}
        for kind, cfg in (("nufapel", n_cfg), ("loselix", l_cfg)):
            model = random_model(registry.config_from_dict(cfg), seed=5, dtype="bf16", device="cuda:0")
            with ClockSampler() as clocks:
                pms = time_prefill(model, PREFILL_TOKENS, warmup=2, reps=5)
                dms, launches, _, _ = time_decode(model, 8, steps, warmup)
            row[kind].update(prefill_tok_s=round(PREFILL_TOKENS / (pms / 1e3), 1), prefill_ms=round(pms, 3),
                             decode_tok_s=round(8 / (dms / 1e3), 1), decode_ms_per_step=round(dms, 4),
                             decode_launches_per_step=launches, clocks=clocks.summary)
            if kind == "loselix":
                lz = dict(z, soft=(z["dim"], z["vdim"], z["dim"] // 2))
                row[kind]["parts"] = design_parts(model, kind, lz, 0, 8, PREFILL_TOKENS, 7, pk)
            else:
                mhz = float(clocks.summary.get("sm_max_mhz") or 1965.0)
                row[kind]["fp32_peak_tflops"] = round(2 * FP32_LANES * mhz * 1e6 / 1e12, 1)
                row[kind]["parts"] = {NUFAPEL_KINDS[i]: nufapel_parts(model, z, i, 8, PREFILL_TOKENS, 7, pk, mhz)
                                      for i in range(min(3, layers))}
            del model
            torch.cuda.empty_cache()
        out["sizes"][tag] = row
    print(json.dumps(out))
    return 0


# ------------------------------------------------------------------ the Gogivik design beside Loselix
# Layer sizes for `--design gogivik`: three layers (chunked attention with rotated values; a state-space layer; latent
# attention with a window and a sink), each over a dense feed-forward and behind input convolutions of three taps,
# beside three Loselix softmax-attention layers of equal width, heads and feed-forward.  "w2k": the width of a 1B-class
# model; "w4k": an 8B-class width.  The latent sizes are those of published latent-attention models (a latent of 512
# with a rotated part of 64, queries through a latent of 1,536), the state-space sizes those of published Mamba-2
# models (heads of 64 values, 128 state channels, four taps).
GOGIVIK_SIZES = {
    "w2k": dict(width=2048, heads=16, kv=4, dim=128, vdim=128, chunk=8192, ssm=(64, 64, 128, 1), lat=(16, 128, 64, 128, 512, 1536),
                window=1024, ff=8192),
    "w4k": dict(width=4096, heads=32, kv=8, dim=128, vdim=128, chunk=8192, ssm=(128, 64, 128, 8), lat=(32, 128, 64, 128, 512, 1536),
                window=1024, ff=16384),
    "small": dict(width=1024, heads=16, kv=4, dim=64, vdim=64, chunk=1536, ssm=(32, 64, 64, 2), lat=(8, 64, 32, 64, 256, 512),
                  window=512, ff=4096),
}
GOGIVIK_KINDS = ("attention", "state_space", "latent_attention")


def gogivik_configs(z, layers, vocab=32000):
    H, G = z["heads"], z["kv"]
    sh, sv, sn, sg = z["ssm"]
    lh, ld, lr, lv, lc, lq = z["lat"]
    dense = {"kind": "dense", "ff": z["ff"]}
    three = [{"type": "attention", "mlp": dense,
              "mixer": {"heads": H, "kv_heads": G, "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
                        "mask": {"size": z["chunk"]}, "rot": {"base": 5e5, "dims": z["dim"], "scaling": {"factor": 8.0}}}},
             {"type": "mamba2", "mlp": dense,
              "mixer": {"heads": sh, "vdim": sv, "state": sn, "groups": sg, "norm_groups": sg, "conv": 4}},
             {"type": "latent_attention", "mlp": dense,
              "mixer": {"heads": lh, "dim": ld, "rot_dim": lr, "vdim": lv, "kv_rank": lc, "q_rank": lq,
                        "scale": (ld + lr) ** -0.5, "mask": {"size": z["window"]}, "rot": {"base": 5e5, "dims": lr}}}]
    gogivik = {"architecture": "Gogivik", "vocab": vocab, "width": z["width"], "norm": {"eps": 1e-5}, "canon": {"taps": 3},
               "logit_scale": 1.0, "layers": [json.loads(json.dumps(three[i % 3])) for i in range(layers)]}
    soft = {"type": "attention_2", "mlp": {"kind": "dense", "ff": z["ff"]},
            "mixer": {"heads": H, "kv_heads": G, "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
                      "rot": {"base": 5e5, "dims": z["dim"] // 2}}}
    loselix = {"architecture": "Loselix", "vocab": vocab, "width": z["width"], "norm": {"eps": 1e-6},
               "layers": [json.loads(json.dumps(soft)) for _ in range(layers)]}
    return gogivik, loselix


def gogivik_parts(model, z, layer_index, batch, tokens, reps, pk, sm_mhz):
    """Layer `layer_index` of a Gogivik model in parts, each alone: the attention kernel (or, for the state-space layer,
    the recurrence from the projected row to the normed heads: convolution, step sizes, scan, gated norm, and the scan
    alone), the preparation of the heads, the input convolution, the whole mixer, the whole feed-forward.  One prompt
    of `tokens` tokens, then one decode step of `batch` requests at CONTEXT tokens.  Rooflines as for the other
    designs; a mask counts: the pairs and the cache rows are those that the chunk or the window lets a query see."""
    import torch
    from jax_vllm_b200 import make_driver, ops
    from jax_vllm_b200.engine import StepEntry
    W = z["width"]
    flush = torch.zeros(160 << 20, dtype=torch.int16, device="cuda")
    layer = model.layers[layer_index]
    mixer, ff = layer.mixer, layer.feed_forward
    kind = GOGIVIK_KINDS[layer_index % 3]
    out = {}

    def seen(pos, mask):                      # keys that a query at `pos` sees
        return pos + 1 if not mask else min(pos + 1, mask) if mask > 0 else pos % (-mask) + 1

    for phase in ("prefill", "decode"):
        if phase == "prefill":
            driver = make_driver(model, max_num_seqs=1, max_model_len=tokens + 16, block_size=PAGE, prefix_cache=False,
                                 max_tokens_per_step=tokens, cuda_graphs=False)
            rc = driver.cache.admit("p")
            driver.cache.grow(rc, tokens)
            entries = [StepEntry(rc, [(i * 7919 + 13) % 1000 for i in range(tokens)], (tokens - 1,))]
            n, seqs, positions = tokens, 1, list(range(tokens))
        else:
            driver = make_driver(model, max_num_seqs=batch, max_model_len=CONTEXT + 64, block_size=PAGE, prefix_cache=False,
                                 cuda_graphs=False)
            rcs = fake_context(driver, batch, CONTEXT)
            for rc in rcs:
                driver.cache.grow(rc, rc.num_tokens + 1)
            entries = [StepEntry(rc, [b], (0,)) for b, rc in enumerate(rcs)]
            n, seqs, positions = batch, batch, [CONTEXT] * batch
        step = driver.runner.builder.build(entries)
        views = driver.runner.layer_caches[layer_index]
        cache, conv_state = layer._split_cache(views)
        x = (torch.randn((n, W), device="cuda") * 0.5).to(torch.bfloat16)
        xf = x.float()
        jobs = []
        bw, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
        if kind == "state_space":
            row = (torch.randn((n, mixer.in_rows), device="cuda") * 0.5).to(torch.bfloat16)
            heads = torch.empty((n, mixer.heads_out), dtype=torch.bfloat16, device="cuda")
            fma = n * mixer.h * mixer.n * mixer.e * 3                          # decay, write, read
            nbytes = seqs * 2 * mixer.h * mixer.n * mixer.e * 4 + n * mixer.in_rows * 2 + n * mixer.heads_out * 2
            roof = (fma / (FP32_LANES * sm_mhz * 1e6) * 1e6, nbytes / bw * 1e6, "fp32 lanes")
            jobs.append(("recurrence", lambda: mixer.from_projection(row, step, cache, heads), roof))
            xbc = (torch.randn((n, mixer.conv_channels), device="cuda") * 0.5).to(torch.bfloat16)
            packed = ops.mamba_prepare(xbc, mixer.inner, mixer.inner + mixer.g * mixer.n, row[:, -mixer.h:], mixer.dt_bias,
                                       mixer.a_log, mixer.h, mixer.g, mixer.n)
            jobs.append(("state scan", lambda: ops.state_scan(packed, xbc, 0, cache.state, step.cu_seqlens, step.state_slots,
                                                              step.n_entries, mixer.e), roof))
            cb = n * mixer.conv_channels * 4 + n * 0
            jobs.append(("mixer convolution", lambda: ops.short_conv(row[:, mixer.inner:mixer.inner + mixer.conv_channels],
                                                                     mixer.conv_w, cache.state[:, mixer.h * mixer.n * mixer.e:],
                                                                     step.cu_seqlens, step.state_slots, step.n_entries,
                                                                     torch.bfloat16, bias=mixer.conv_b, act="silu"),
                         (0.0, cb / bw * 1e6, "flops")))
        else:
            table = step.block_tables[cache.group]
            mask = mixer.mask
            pairs = sum(seen(p, mask) for p in positions)
            if phase == "prefill":
                keys = tokens
            else:
                keys = batch * seen(CONTEXT, mask)
            if kind == "attention":
                q = torch.randn((n, mixer.hq * mixer.d), device="cuda").to(torch.bfloat16)
                a = torch.empty((n, mixer.hq * mixer.dv), dtype=torch.bfloat16, device="cuda")
                attn = lambda: mixer.attend(q, a, step, cache, table)
                flops = 2 * mixer.hq * (mixer.d + mixer.dv) * pairs
                nbytes = keys * (mixer.hk * mixer.d + mixer.hv * mixer.dv) * 2 + n * mixer.hq * (mixer.d + mixer.dv) * 2
                rowp = (torch.randn((n, mixer.in_rows), device="cuda") * 0.5).to(torch.bfloat16)
                prep = lambda: ops.head_prepare(rowp, 0, mixer.k_off, mixer.v_off, q, step.positions, step.token_entry, table,
                                                mixer.position.table(), False, mixer.q_norm, mixer.k_norm, 1e-5, True,
                                                mixer.value_freq, cache.k, cache.v, mixer.hq, mixer.hk, mixer.hv, mixer.d, mixer.dv)
                pb = n * mixer.in_rows * 2 * 2
                jobs.append(("head preparation", prep, (0.0, pb / bw * 1e6, "flops")))
                jobs.append(("output rotation", lambda: ops.head_rotate(a, step.positions, mixer.value_freq, False, mixer.h,
                                                                        mixer.dv, sign=-1.0),
                             (0.0, n * mixer.hq * mixer.dv * 4 / bw * 1e6, "flops")))
            else:
                q = torch.randn((n, mixer.h * mixer.dk), device="cuda").to(torch.bfloat16)
                attn = lambda: mixer.attend(q, step, cache, table)
                flops = 2 * mixer.h * (mixer.dk + mixer.dc) * pairs
                nbytes = keys * mixer.dk * 2 + n * mixer.h * (mixer.dk + mixer.dc) * 2
            jobs.append(("attention kernel", attn, (flops / tf * 1e6, nbytes / bw * 1e6, "flops")))
        if conv_state[0] is not None:
            jobs.append(("input convolution", lambda: ops.short_conv(xf, layer.conv_w[0], conv_state[0].state, step.cu_seqlens,
                                                                     step.state_slots, step.n_entries, torch.bfloat16,
                                                                     residual=True), (0.0, n * W * 6 / bw * 1e6, "flops")))
        jobs.append(("mixer", lambda: mixer.forward(x, step, cache), None))
        ff_flops, ff_bytes = 2 * n * 2 * z["ff"] * W, 2 * z["ff"] * W * 2
        jobs.append(("feed-forward", lambda: ff.forward(x, step), (ff_flops / tf * 1e6, ff_bytes / bw * 1e6, "flops")))
        res = {}
        for name, fn, roof in jobs:
            us = time_part(fn, reps, flush)
            res[name] = {"us": round(us, 1)}
            if roof is not None:
                t_math, t_bytes, unit = roof
                ideal = max(t_math, t_bytes)
                res[name].update(roofline_us=round(ideal, 1), bound=unit if t_math >= t_bytes else "bytes",
                                 of_roofline=round(ideal / us, 3))
        driver.runner.check_kernels()
        out[phase] = res
        del driver
        torch.cuda.empty_cache()
    return out


def design_gogivik(layers, sizes, steps, warmup) -> int:
    import torch
    from jax_vllm_b200 import random_model, registry
    pk, pk_src = peaks()
    sizes = [t for t in sizes if t in GOGIVIK_SIZES] or ["w2k", "w4k"]
    out = {"design": "gogivik", "layers": layers, "prefill_tokens": PREFILL_TOKENS, "decode_batch": 8, "context": CONTEXT,
           "dtype": "bf16", "data": "synthetic (random weights, seed 5)", "peaks": pk, "peak_source": pk_src, "sizes": {}}
    for tag in sizes:
        z = GOGIVIK_SIZES[tag]
        g_cfg, l_cfg = gogivik_configs(z, layers)
        row = {"gogivik": {"config": {k: v for k, v in z.items()}},
               "loselix": {"config": {"width": z["width"], "heads": z["heads"], "kv": z["kv"], "dim": z["dim"], "ff": z["ff"]}}}
        for kind, cfg in (("gogivik", g_cfg), ("loselix", l_cfg)):
            model = random_model(registry.config_from_dict(cfg), seed=5, dtype="bf16", device="cuda:0")
            with ClockSampler() as clocks:
                pms = time_prefill(model, PREFILL_TOKENS, warmup=2, reps=5)
                dms, launches, _, _ = time_decode(model, 8, steps, warmup)
            row[kind].update(prefill_tok_s=round(PREFILL_TOKENS / (pms / 1e3), 1), prefill_ms=round(pms, 3),
                             decode_tok_s=round(8 / (dms / 1e3), 1), decode_ms_per_step=round(dms, 4),
                             decode_launches_per_step=launches, clocks=clocks.summary)
            if kind == "loselix":
                lz = dict(z, soft=(z["dim"], z["vdim"], z["dim"] // 2))
                row[kind]["parts"] = design_parts(model, kind, lz, 0, 8, PREFILL_TOKENS, 7, pk)
            else:
                mhz = float(clocks.summary.get("sm_max_mhz") or 1965.0)
                row[kind]["fp32_peak_tflops"] = round(2 * FP32_LANES * mhz * 1e6 / 1e12, 1)
                row[kind]["parts"] = {GOGIVIK_KINDS[i]: gogivik_parts(model, z, i, 8, PREFILL_TOKENS, 7, pk, mhz)
                                      for i in range(min(3, layers))}
            del model
            torch.cuda.empty_cache()
        out["sizes"][tag] = row
    print(json.dumps(out))
    return 0


def reference_arm():
    why = ("the reference (jllm) needs jax, jaxlib and equinox and the hatchling build backend; none is installed "
           "and none is in the offline wheelhouse, so it can neither be installed nor run here")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the configuration has (same layer sizes), for a quick run")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64, and the prefill")
    ap.add_argument("--only-prefill", action="store_true", help="time the 2,048-token prefill alone (for profiling)")
    ap.add_argument("--micro", default=None, help="run one kernel alone, e.g. linear:24576x4096:8 (see micro())")
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="a serving workload of a larger shape through the entry point (see WORKLOADS); --layers cuts it")
    ap.add_argument("--timeline", type=int, default=None, metavar="BATCH",
                    help="print every kernel of one replayed decode step at this batch with its start and end (use --layers)")
    ap.add_argument("--with-workloads", action="store_true",
                    help="after the headline run, also run the two serving workloads and add their lines under `workloads`")
    ap.add_argument("--design", default=None, metavar="NAME",
                    help="guronex, loselix, nufapel or gogivik: that design's prefill and decode throughput at a few layer sizes "
                         "beside its closest neighbour of equal size (Qwen3; for nufapel, Loselix), with the rooflines of "
                         "its kernels (see design())")
    ap.add_argument("--sizes", default="lite,mid,row576",
                    help="with --design: which of its layer sizes, comma-separated (guronex: lite,mid,row576; loselix: "
                         "w2k,w4k,mix, all by default; nufapel and gogivik: w2k,w4k,small, the first two by default)")
    ap.add_argument("--micro-eager", action="store_true",
                    help="with --micro: plain launches instead of replays of a CUDA graph (for a profiler)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.micro:
        return micro(args.micro, max(1, args.steps), args.micro_eager)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.design:
        return design(args.design, args.layers, [t for t in args.sizes.split(",") if t], max(8, args.steps // 2),
                      max(3, args.warmup))
    if args.timeline:
        return timeline(args.timeline, args.layers or 4, args.workload)
    if args.workload:
        return workload(args.workload, args.layers)
    args.layers = args.layers or QWEN3_8B["num_hidden_layers"]
    warmup = max(3, args.warmup)

    import torch
    from jax_vllm_b200 import random_model, registry

    cfg_dict = dict(QWEN3_8B, num_hidden_layers=args.layers)
    cfg = registry.config_from_dict(cfg_dict)
    model = random_model(cfg, seed=5, dtype="bf16", device="cuda:0")
    pk, pk_src = peaks()
    if args.only_prefill:
        pms = time_prefill(model, PREFILL_TOKENS, warmup=1, reps=max(1, args.steps))
        print(json.dumps({"prefill_ms": round(pms, 3), "tokens": PREFILL_TOKENS, "layers": args.layers}))
        return 0

    region_clocks = {}
    with ClockSampler() as clocks:
        ms, launches, repeats, all_ms = time_decode(model, args.batch, args.steps, warmup)
    region_clocks["decode"] = clocks.summary
    value = args.batch / (ms / 1e3)
    bytes_step = decode_bytes(cfg_dict, args.layers, args.batch, CONTEXT + warmup + repeats * args.steps // 2)
    achieved = bytes_step / (ms / 1e3) / 1e9
    out = {
        "metric": f"decode tok/s (Qwen3-8B shape, bf16, batch {args.batch}, {CONTEXT}-token context)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "repeats": repeats, "ms_per_step_of_repeats": [round(v, 4) for v in all_ms],
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (uniform random token ids, random N(0,0.02) weights, seed 5)",
        "config": {"model": "Qwen3-8B shape", "layers": args.layers, "layers_of_config": QWEN3_8B["num_hidden_layers"],
                   "hidden": 4096, "q_heads": 32, "kv_heads": 8, "head_dim": 128, "intermediate": 12288,
                   "vocab": 151936, "global_batch": args.batch, "seq_len": CONTEXT, "max_context": 4096,
                   "page_size": PAGE, "parallelism": "none (1 GPU)", "l2": "inputs larger than L2 (15 GB of weights)",
                   "cuda_graphs": True, "timed": f"median of {repeats} repeats of {args.steps} steps"},
        "gpu_launches": launches * args.steps * repeats,
        "clocks": clocks.summary,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk_src},
    }
    if not args.skip_points:
        with ClockSampler() as c:
            e2e, e2e_best, runs, h2d, d2h = time_e2e(model, args.batch, args.steps, warmup)
        region_clocks["e2e"] = c.summary
        out["e2e"] = {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                      "runs": runs, "picked": "median over the runs of `steps` steps", "best": round(e2e_best, 1)}
        with ClockSampler() as c:
            pms = time_prefill(model, PREFILL_TOKENS, warmup=2, reps=max(3, int(MIN_TIMED_SECONDS / 0.027)))
        region_clocks["prefill"] = c.summary
        flops = prefill_flops(cfg_dict, args.layers, PREFILL_TOKENS)
        out["prefill"] = {"value": round(PREFILL_TOKENS / (pms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pms, 3),
                          "frac": round(flops / (pms / 1e3) / 1e12 / pk["bf16_tflops"], 4),
                          "peak_tflops": pk["bf16_tflops"], "peak_source": pk_src}
        points = {}
        for b in (1, 64):
            with ClockSampler() as c:
                pms_b, _, _, _ = time_decode(model, b, max(8, args.steps // 2), warmup)
            region_clocks[f"decode_b{b}"] = c.summary
            points[f"decode_b{b}"] = round(b / (pms_b / 1e3), 1)
            frac = decode_bytes(cfg_dict, args.layers, b, CONTEXT + 64) / (pms_b / 1e3) / 1e9 / pk["hbm_gbs"]
            points[f"decode_b{b}_hbm_frac"] = round(frac, 4)
        out["points"] = points
    out["clocks_by_region"] = region_clocks
    if args.with_workloads:
        # the two serving workloads of larger shapes, each in a process of its own (they need the device's memory)
        del model
        torch.cuda.empty_cache()
        out["workloads"] = {}
        for name in sorted(WORKLOADS):
            proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--workload", name], capture_output=True, text=True)
            line = [l for l in proc.stdout.splitlines() if l.startswith("{")]
            out["workloads"][name] = json.loads(line[-1]) if proc.returncode == 0 and line else {"failed": proc.stderr[-300:]}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
