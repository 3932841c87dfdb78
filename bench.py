#!/usr/bin/env python3
"""Benchmark of the engine's decode step (and prefill) on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default workload: the layer sizes of Qwen3-0.6B (configs/qwen3-0.6b.json) with random
weights, bfloat16, 8 requests decoding at a context of 4,096 tokens, pages of 16 tokens.
One "step" is one decode step: every live request advances by one token (step function,
then the sampling kernel).  One JSON line is printed:

* ``value``: decoded tokens a second over exactly K steps, timed with CUDA events on the
  launching stream, after W warm-up steps, with a synchronize on both sides;
* ``e2e``: the same through the public ``Engine`` API: every step copies the step's token
  ids and tables from pinned host memory to the device and reads the sampled token ids back;
* ``prefill``: one prompt of 2,048 tokens in one step: tokens a second, milliseconds, and the
  fraction of the tensor-core peak that the step's flops amount to;
* ``roofline``: bytes a decode step has to read (every weight it uses once, and the keys and
  values of the live requests) over its time, against the measured copy bandwidth;
* ``points``: decode tokens a second at batch 1 and 64 (same context);
* ``clocks``: SM clock and throttle reasons sampled with nvidia-smi during the timed region.

The contexts are synthetic: the pages of each request are filled with random keys and values
instead of being computed by a prefill, which changes nothing of what a decode step reads
or computes.  Inputs are larger than the L2 cache (weights 1.2 GB, keys and values 3.8 GB),
so no L2 flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0          # copy bandwidth measured earlier on this pool
FALLBACK_BF16_TFLOPS = 1590.0      # cuBLAS bf16 burst measured earlier on this pool
CONTEXT = 4096
PREFILL_TOKENS = 2048


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm, tf, src = FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"
    try:
        with open(path) as f:
            d = json.load(f)
        got_hbm, got_tf = d.get("hbm_gbs"), d.get("bf16_tflops")
        if isinstance(got_hbm, (int, float)) and got_hbm > 0 and isinstance(got_tf, (int, float)) and got_tf > 0:
            hbm, tf, src = float(got_hbm), float(got_tf), "measured"
    except (OSError, ValueError, TypeError, AttributeError):
        pass
    return hbm, tf, src


class ClockSampler:
    """nvidia-smi in the background, every 50 ms, while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def fill_contexts(runner, batch, context, prefix="c"):
    """``batch`` live requests that hold ``context`` tokens of random keys and values."""
    import torch
    cache = runner.cache
    rids = []
    for i in range(batch):
        rid = f"{prefix}{i}"
        cache.add_request(rid)
        cache.allocate(rid, context)
        cache.commit(rid, context)
        rids.append(rid)
    return rids


def randomize_pages(runner, seed=0):
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    for grp in runner.cache.kv_groups:
        for t in grp.tensors.values():
            flat = t.view(-1)
            step = 1 << 26
            for s in range(0, flat.numel(), step):
                chunk = flat[s:s + step]
                chunk.copy_(torch.randn(chunk.numel(), generator=g, device="cuda", dtype=torch.float32).mul_(0.5))


def release(runner, rids):
    for rid in rids:
        runner.cache.free_request(rid)


def decode_bytes(plan, runner, contexts, weight_esize):
    """Bytes one decode step must read: each weight it uses once and the live keys and values."""
    t = plan.tensors()
    skip = set()
    if not plan.lm_head.tied:
        skip.add(plan.embedding.weight)           # an untied embedding is only gathered from
    w = 0
    for name, spec in t.items():
        if name in skip:
            continue
        n = 1
        for s in spec.shape:
            n *= s
        w += n * weight_esize
    kv = sum(contexts) * runner.cache.bytes_per_token()
    return w, kv


def prefill_flops(cfg, tokens):
    h, i, nq, nkv, d, L = (cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                           cfg.head_dim, cfg.num_hidden_layers)
    per_token = 2 * (h * (nq + 2 * nkv) * d + nq * d * h + 3 * h * i)
    linear = L * per_token * tokens
    attn = L * 4 * nq * d * tokens * (tokens + 1) // 2
    head = 2 * h * cfg.vocab_size
    return linear + attn + head


def time_decode(runner, rids, vocab, steps, warmup, seed=1):
    """Device time of ``steps`` decode steps (ms), each step: step function + sampling kernel."""
    import torch
    from infurnace_b200.engine.runner import StepEntry
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, vocab, (warmup + steps, len(rids)), generator=g).tolist()
    zeros = [0.0] * len(rids)

    def one(k):
        # the step function with the sampling kernel behind it; decode-only steps replay a CUDA graph
        runner.step_and_sample([StepEntry(rid, [ids[k][j]], [0]) for j, rid in enumerate(rids)], zeros, zeros)

    for k in range(warmup):
        one(k)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = runner.rt.kernels.launches
    replays0 = runner.graph_replays
    start.record()
    for k in range(warmup, warmup + steps):
        one(k)
    end.record()
    torch.cuda.synchronize()
    launches = runner.rt.kernels.launches - launches0
    replays = runner.graph_replays - replays0
    if replays:          # a replayed step launches what one recorded step launched
        launches += replays * runner.launches_per_graph_step
    return start.elapsed_time(end), launches


def run_ours(args):
    import torch
    from infurnace_b200.engine import Engine, EngineOptions, Request, SamplingParams
    from infurnace_b200.engine.runner import StepEntry
    from infurnace_b200.models import read_config
    from infurnace_b200.weights.random_init import write_random_model

    hbm_peak, tf_peak, peak_src = read_peaks()
    cfg = read_config(os.path.join(ROOT, "configs", "qwen3-0.6b.json"))
    batch, steps, warmup = args.batch, args.steps, args.warmup
    layers_full = cfg.num_hidden_layers
    page = args.page_size
    big = 64 if args.mode == "all" else batch          # the largest batch of the run
    pool_tokens = big * CONTEXT + PREFILL_TOKENS + 64
    with tempfile.TemporaryDirectory(prefix="infurnace_b200_bench_") as d:
        write_random_model(cfg, 0, d)
        opts = EngineOptions(dtype="bfloat16", page_size=page, num_pages=pool_tokens // page, max_num_seqs=big,
                             max_num_batched_tokens=PREFILL_TOKENS, max_model_len=CONTEXT)
        engine = Engine.from_model_dir(d, opts)
    runner, plan = engine.runner, engine.plan
    if args.eager:
        runner.use_graphs = False
    if args.mode == "prefill":
        toks = torch.randint(0, cfg.vocab_size, (PREFILL_TOKENS,)).tolist()
        times = []
        for rep in range(max(1, steps)):
            runner.cache.add_request("p")
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            s.record()
            runner.step([StepEntry("p", toks, [PREFILL_TOKENS - 1])])
            e.record()
            torch.cuda.synchronize()
            runner.cache.free_request("p")
            times.append(s.elapsed_time(e))
        print(json.dumps({"mode": "prefill", "tokens": PREFILL_TOKENS, "steps": max(1, steps),
                          "ms_median": statistics.median(times), "ms_min": min(times)}))
        return 0
    randomize_pages(runner)
    torch.cuda.synchronize()
    start_ctx = CONTEXT - warmup - steps

    # ---- decode, device timed
    clocks = ClockSampler()
    rids = fill_contexts(runner, batch, start_ctx)
    clocks.start()
    ms, launches = time_decode(runner, rids, cfg.vocab_size, steps, warmup)
    clock_report = clocks.stop()
    release(runner, rids)
    ms_per_step = ms / steps
    value = batch * steps / (ms / 1000.0)
    if args.mode == "decode":
        print(json.dumps({"mode": "decode", "batch": batch, "context": CONTEXT, "steps": steps, "ms_per_step": ms_per_step,
                          "tokens_per_s": value, "graphs": runner.use_graphs, "launches": launches}))
        return 0
    mean_ctx = CONTEXT - steps / 2
    w_bytes, kv_bytes = decode_bytes(plan, runner, [mean_ctx] * batch, 2)
    achieved = (w_bytes + kv_bytes) / (ms_per_step / 1000.0) / 1e9

    # ---- decode, end to end through the Engine API (host token ids in and out every step)
    e2e = time_e2e(engine, cfg.vocab_size, batch, steps, warmup)

    # ---- prefill of 2,048 tokens in one step
    toks = torch.randint(0, cfg.vocab_size, (PREFILL_TOKENS,)).tolist()
    times = []
    for rep in range(2 + 3):
        runner.cache.add_request("p")
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        runner.step([StepEntry("p", toks, [PREFILL_TOKENS - 1])])
        e.record()
        torch.cuda.synchronize()
        runner.cache.free_request("p")
        if rep >= 2:
            times.append(s.elapsed_time(e))
    pre_ms = statistics.median(times)
    flops = prefill_flops(cfg, PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / (pre_ms / 1000.0), "tokens": PREFILL_TOKENS, "ms": pre_ms,
               "frac": flops / (pre_ms / 1000.0) / (tf_peak * 1e12), "tflops": flops / (pre_ms / 1000.0) / 1e12,
               "peak_tflops": tf_peak, "peak_source": peak_src}

    # ---- other batch sizes
    points = {}
    for b in (1, 64):
        k = max(8, steps // 2)
        rids = fill_contexts(runner, b, CONTEXT - warmup - k)
        pms, _ = time_decode(runner, rids, cfg.vocab_size, k, warmup)
        release(runner, rids)
        points[f"decode_b{b}"] = b * k / (pms / 1000.0)

    line = {
        "metric": f"decode tok/s at batch {batch}, context {CONTEXT} (Qwen3-0.6B shape, random weights)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"model": "Qwen3-0.6B shape, random weights seed 0", "layers": layers_full, "layers_run": layers_full,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": batch, "seq_len": CONTEXT, "page_size": page, "prefill_tokens": PREFILL_TOKENS,
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (weights 1.2 GB + KV)",
                   "context_fill": "random keys/values in pages"},
        "e2e": e2e, "gpu_launches": launches, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "bytes_per_step": w_bytes + kv_bytes, "peak_source": peak_src},
        "points": points, "clocks": clock_report,
    }
    print(json.dumps(line))
    return 0


def time_e2e(engine, vocab, batch, steps, warmup):
    """Decode through Engine.step(): scheduler, pinned host staging, H2D copy, kernels, sampling,
    and the read-back of the sampled ids, every step.  The contexts are real here: the prompts
    are prefilled through the same engine first (not timed)."""
    import torch
    from infurnace_b200.engine import Request, RequestState, SamplingParams
    # requests that finish their prompt early decode while the others still prefill: leave room for that
    prefill_steps = -(-batch * CONTEXT // engine.runner.max_tokens) + 2
    budget = warmup + steps + 2 + prefill_steps
    prompts = torch.randint(0, vocab, (batch, CONTEXT - budget), generator=torch.Generator().manual_seed(3)).tolist()
    reqs = [Request(f"e{j}", prompts[j], SamplingParams(max_tokens=budget)) for j in range(batch)]
    for r in reqs:
        engine.add_request(r)
    guard = 0
    while any(r.state is not RequestState.DECODING for r in reqs):
        engine.step()
        guard += 1
        if guard > 10000 or any(r.is_terminal() for r in reqs):
            raise RuntimeError("prefill for the end-to-end measurement did not complete")
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    s.record()
    n = 0
    for _ in range(steps):
        n += engine.step().num_decode_tokens
    e.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    for r in reqs:
        engine.cancel(r.request_id)
    run = engine.runner
    h2d = run._small_len * 4 + batch * run.max_pages * 4 * max(1, len(run.cache.kv_groups))
    return {"value": n / wall, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": batch * 4,
            "ms_per_step": wall * 1000 / steps, "device_ms_per_step": s.elapsed_time(e) / steps}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--page-size", type=int, default=16, help="tokens per page of the key/value cache")
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--mode", default="all", choices=("all", "decode", "prefill"),
                    help="decode / prefill: only that part, on a pool just large enough (for profiling a small case)")
    ap.add_argument("--eager", action="store_true", help="launch every kernel of a decode step instead of replaying a graph")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference's model and runner import tinygrad, which is not installed and has no wheel "
                          "offline (pip install --no-deps succeeds, import infurnace.executor.tinygrad.model fails)"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(3, args.warmup)
    return run_ours(args)


if __name__ == "__main__":
    raise SystemExit(main())
