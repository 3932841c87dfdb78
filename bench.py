#!/usr/bin/env python3
"""Benchmark of the engine's decode step (and prefill) on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config configs/qwen3-0.6b.json] [--layers N] [--batch 8] [--context 4096]

Default workload: the layer sizes of Qwen3-0.6B (configs/qwen3-0.6b.json) with random weights
drawn on the device, bfloat16, 8 requests decoding at a context of 4,096 tokens, pages of 16
tokens.  ``--config`` names another configuration of the architecture (configs/qwen3-8b.json,
configs/qwen3-32b.json); ``--layers`` runs fewer layers than it has (``config`` in the output names
both numbers).  One "step" is one decode step: every live request advances by one token (step
function, then the sampling kernel).  One JSON line is printed:

* ``value``: decoded tokens a second over exactly K steps, timed with CUDA events on the
  launching stream, after W warm-up steps, with a synchronize on both sides; ``samples``: the
  smallest, mean and median step time from an event after every step (the reference's
  ``timing_summary``, benchmarks/common.py:44-53);
* ``e2e``: the same through the public ``Engine`` API: every step copies the step's token
  ids and tables from pinned host memory to the device and reads the sampled token ids back;
* ``prefill``: one prompt of 2,048 tokens in one step: tokens a second, milliseconds, and the
  fraction of the tensor-core peak that the step's flops amount to;
* ``roofline``: bytes a decode step has to read (every weight it uses once, and the keys and
  values of the live requests) over its time, against the measured copy bandwidth;
* ``points``: decode tokens a second at batch 1 and 64 (same context), and ``gen_b1/8/64``: the
  reference's closed loop (benchmarks/benchmark_decode.py:24-33, tools/run_infurnace_model.py:19-44):
  prompts of 128 tokens prefilled through the engine, then 256 tokens generated greedily through
  ``Engine.step()``, tokens a second over the decode steps; ``points_detail`` gives each point's
  microseconds per step (min / mean / median) and its fraction of the HBM bound;
* ``kernels``: where a decode step's and the prefill's time goes by class of kernel (attention,
  products, LM head, the rest), from an eager pass with CUDA events around every launch
  (launches then do not overlap their neighbours, so the classes add up to more than the
  graph-replayed step: compare shares), with each class's achieved GB/s or TFLOP/s;
* ``clocks``: SM clock and throttle reasons sampled with nvidia-smi during the timed region.

The contexts of the device-timed decode steps are synthetic: the pages of each request are filled
with random keys and values instead of being computed by a prefill, which changes nothing of what
a decode step reads or computes.  Inputs are larger than the L2 cache (weights 1.2 GB and more, keys
and values 3.8 GB and more at the default), so no L2 flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0          # copy bandwidth of a B200, used when no measured figure is at hand
FALLBACK_BF16_TFLOPS = 1590.0      # library bf16 matrix-product burst of a B200, likewise
PREFILL_TOKENS = 2048
GEN_PROMPT, GEN_TOKENS = 128, 256


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


def summary(ms):
    """min / mean / median of a list of times in milliseconds."""
    return {"min_ms": min(ms), "mean_ms": statistics.fmean(ms), "median_ms": statistics.median(ms), "n": len(ms)}


def fill_contexts(runner, batch, context, prefix="c"):
    """``batch`` live requests that hold ``context`` tokens of (random) keys and values."""
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
        tensors = [t for t in grp.tensors.values() if t is not None]
        tensors += [x for cid, t in grp.tensors.items() if t is None for x in grp.streams[cid].values()]
        for t in tensors:
            flat = t.view(-1)
            step = 1 << 26
            for s in range(0, flat.numel(), step):
                chunk = flat[s:s + step]
                chunk.copy_(torch.randn(chunk.numel(), generator=g, device="cuda", dtype=torch.float32).mul_(0.5))


def release(runner, rids):
    for rid in rids:
        runner.cache.free_request(rid)


def weight_bytes(plan, esize):
    """Bytes of every tensor a decode step reads once (an untied embedding is only gathered from)."""
    skip = set() if plan.lm_head.tied else {plan.embedding.weight}
    total = 0
    for name, spec in plan.tensors().items():
        if name in skip:
            continue
        n = 1
        for s in spec.shape:
            n *= s
        total += n * esize
    return total


def decode_bytes(plan, runner, contexts, esize):
    """Bytes one decode step must read: each weight it uses once and the live keys and values."""
    return weight_bytes(plan, esize), sum(contexts) * runner.cache.bytes_per_token()


def prefill_flops(plan, tokens):
    """Flops of one prompt of ``tokens`` tokens in one step, from the plan: two per weight element and
    token for every matrix of every layer call, causal attention scores and values (window honoured),
    and the head on the one wanted row."""
    linear = attn = 0
    for call in plan.resolved_schedule():
        layer = plan.layers[call.layer]
        for spec in layer.tensors().values():
            if len(spec.shape) == 2:
                linear += 2 * spec.shape[0] * spec.shape[1] * tokens
        mixer = getattr(layer, "mixer", None)
        heads, hd = getattr(mixer, "num_heads", None), getattr(mixer, "head_dim", None)
        if heads and hd:
            w = getattr(mixer, "window", None)
            pairs = tokens * (tokens + 1) // 2 if not w or w >= tokens else w * (w + 1) // 2 + (tokens - w) * w
            attn += 4 * heads * hd * pairs
    head = 2 * plan.hidden_size * plan.vocab_size
    return linear + attn + head


def hold_the_device(ms=12.0):
    """Keep the device busy for about ``ms`` so that the launches that follow queue up behind it: the events
    around them then measure the kernels, not the host's time between launches."""
    import torch
    torch.cuda._sleep(int(ms * 1.9e6))


class KernelClassTimer:
    """CUDA events around every launch of the kernel set, by class.  With events between them, launches do
    not overlap their neighbours (no programmatic dependent launch), so times are those of kernels alone
    on a warm device; the caller queues the launches behind ``hold_the_device`` so that the host's pace
    does not show."""
    METHODS = ("embed", "rmsnorm", "linear", "linear_residual_norm", "rope_table", "qk_norm_rope_store",
               "paged_attention", "sample")

    def __init__(self, kernels, vocab):
        self.k, self.vocab = kernels, vocab
        self.records = []          # (class, start event, end event, bytes, flops)
        self.kv_bytes_per_call = 0
        self.attn_flops_per_call = 0
        self._saved = {}

    def __enter__(self):
        import torch
        for name in self.METHODS:
            inner = getattr(self.k, name)
            self._saved[name] = inner

            def wrapped(*a, _inner=inner, _name=name, **kw):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                out = _inner(*a, **kw)
                e.record()
                self.records.append((*self._classify(_name, a, kw), s, e))
                return out
            setattr(self.k, name, wrapped)
        return self

    def __exit__(self, *exc):
        for name, inner in self._saved.items():
            setattr(self.k, name, inner)
        return False

    def _classify(self, name, a, kw):
        if name == "paged_attention":
            return "attention", self.kv_bytes_per_call, self.attn_flops_per_call
        if name in ("linear", "linear_residual_norm"):
            x, w = a[0], a[1]
            cls = "lm_head" if w.shape[0] == self.vocab else "products"
            return cls, w.numel() * w.element_size(), 2 * x.shape[0] * w.numel()
        return "rest", 0, 0

    def report(self, steps):
        import torch
        torch.cuda.synchronize()
        out = {}
        for cls, nbytes, flops, s, e in self.records:
            d = out.setdefault(cls, {"ms": 0.0, "bytes": 0, "flops": 0, "launches": 0})
            d["ms"] += s.elapsed_time(e)
            d["bytes"] += nbytes
            d["flops"] += flops
            d["launches"] += 1
        total = sum(d["ms"] for d in out.values()) or 1.0
        rep = {}
        for cls, d in out.items():
            r = {"ms_per_step": d["ms"] / steps, "share": d["ms"] / total, "launches_per_step": d["launches"] // steps}
            if d["bytes"]:
                r["gbs"] = d["bytes"] / (d["ms"] / 1000.0) / 1e9
            if d["flops"]:
                r["tflops"] = d["flops"] / (d["ms"] / 1000.0) / 1e12
            rep[cls] = r
        return rep


def time_decode(runner, rids, vocab, steps, warmup, seed=1):
    """Device time of ``steps`` decode steps (ms), each step: step function + sampling kernel; and the
    time of each step from an event recorded after it."""
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
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    launches0 = runner.rt.kernels.launches
    replays0 = runner.graph_replays
    marks[0].record()
    for k in range(steps):
        one(warmup + k)
        marks[k + 1].record()
    torch.cuda.synchronize()
    launches = runner.rt.kernels.launches - launches0
    replays = runner.graph_replays - replays0
    if replays:          # a replayed step launches what one recorded step launched
        launches += replays * runner.launches_per_graph_step
    per_step = [marks[k].elapsed_time(marks[k + 1]) for k in range(steps)]
    return marks[0].elapsed_time(marks[steps]), launches, per_step


def time_prefill(runner, vocab, reps, warm=2):
    import torch
    from infurnace_b200.engine.runner import StepEntry
    toks = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=torch.Generator().manual_seed(2)).tolist()
    times = []
    for rep in range(warm + reps):
        runner.cache.add_request("p")
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        runner.step([StepEntry("p", toks, [PREFILL_TOKENS - 1])])
        e.record()
        torch.cuda.synchronize()
        runner.cache.free_request("p")
        if rep >= warm:
            times.append(s.elapsed_time(e))
    return times


def profile_classes(runner, plan, cfg_sizes, batch, context, vocab, esize):
    """The eager pass: kernel classes of a decode step at (batch, context) and of the 2,048-token prefill."""
    import torch
    from infurnace_b200.engine.runner import StepEntry
    K = runner.rt.kernels
    graphs = runner.use_graphs
    runner.use_graphs = False
    out = {}
    try:
        steps = 3
        rids = fill_contexts(runner, batch, context - steps - 2, prefix="k")
        zeros = [0.0] * batch
        step = lambda: runner.step_and_sample([StepEntry(r, [1], [0]) for r in rids], zeros, zeros)      # noqa: E731
        step(); step()
        with KernelClassTimer(K, vocab) as t:
            t.kv_bytes_per_call = batch * context * cfg_sizes["kv_bytes_per_token_per_layer"]
            for _ in range(steps):
                torch.cuda.synchronize()
                hold_the_device()
                step()
            out["decode"] = t.report(steps)
        release(runner, rids)
        toks = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=torch.Generator().manual_seed(2)).tolist()
        for rep in range(2):
            runner.cache.add_request("kp")
            if rep == 1:
                with KernelClassTimer(K, vocab) as t:
                    t.attn_flops_per_call = cfg_sizes["attn_flops_per_layer_prefill"]
                    torch.cuda.synchronize()
                    hold_the_device(20.0)
                    runner.step([StepEntry("kp", toks, [PREFILL_TOKENS - 1])])
                    out["prefill"] = t.report(1)
            else:
                runner.step([StepEntry("kp", toks, [PREFILL_TOKENS - 1])])
            runner.cache.free_request("kp")
    finally:
        runner.use_graphs = graphs
    for phase in out.values():
        for cls, r in phase.items():
            for key in list(r):
                if isinstance(r[key], float):
                    r[key] = round(r[key], 4)
    return out


def time_generation(engine, plan, vocab, batch, hbm_peak, esize, seed=5):
    """The reference's closed loop: ``batch`` prompts of 128 tokens prefilled through the engine, then 256
    tokens each generated greedily through ``Engine.step()`` (no end-of-sequence id: every request runs to
    its count).  Timed: the decode steps from the moment every request decodes, host clock around each
    ``step()`` (plan, staging copy, kernels, read-back of the tokens)."""
    import torch
    from infurnace_b200.engine import Request, RequestState, SamplingParams
    prompts = torch.randint(0, vocab, (batch, GEN_PROMPT), generator=torch.Generator().manual_seed(seed)).tolist()
    reqs = [Request(f"g{batch}-{j}", prompts[j], SamplingParams(max_tokens=GEN_TOKENS)) for j in range(batch)]
    for r in reqs:
        engine.add_request(r)
    guard = 0
    while any(r.state is not RequestState.DECODING for r in reqs):
        engine.step()
        guard += 1
        if guard > 1000 or any(r.is_terminal() for r in reqs):
            raise RuntimeError("prefill for the generation measurement did not complete")
    for _ in range(3):
        engine.step()
    torch.cuda.synchronize()
    left = min(r.sampling_params.max_tokens - len(r.output_token_ids) for r in reqs) - 2
    times, tokens = [], 0
    start_ctx = statistics.fmean(r.num_tokens for r in reqs)
    t_all = time.perf_counter()
    for _ in range(left):
        t0 = time.perf_counter()
        tokens += engine.step().num_decode_tokens
        times.append((time.perf_counter() - t0) * 1000.0)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t_all
    end_ctx = statistics.fmean(r.num_tokens for r in reqs)
    while not engine.is_done():
        engine.step()
    w = weight_bytes(plan, esize)
    kv = batch * (start_ctx + end_ctx) / 2 * engine.runner.cache.bytes_per_token()
    bound_us = (w + kv) / (hbm_peak * 1e9) * 1e6
    s = summary(times)
    return {"tokens_per_s": tokens / wall, "steps": left, "us_per_step_min": s["min_ms"] * 1000, "us_per_step_mean": wall / left * 1e6,
            "us_per_step_median": s["median_ms"] * 1000, "bound_us": bound_us, "frac": bound_us / (wall / left * 1e6),
            "mean_context": (start_ctx + end_ctx) / 2}


def time_e2e(engine, vocab, batch, context, steps, warmup):
    """Decode through Engine.step(): scheduler, pinned host staging, H2D copy, kernels, sampling,
    and the read-back of the sampled ids, every step.  The contexts are real here: the prompts
    are prefilled through the same engine first (not timed)."""
    import torch
    from infurnace_b200.engine import Request, RequestState, SamplingParams
    # requests that finish their prompt early decode while the others still prefill: leave room for that
    prefill_steps = -(-batch * context // engine.runner.max_tokens) + 2
    budget = warmup + steps + 2 + prefill_steps
    prompts = torch.randint(0, vocab, (batch, context - budget), generator=torch.Generator().manual_seed(3)).tolist()
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
    while not engine.is_done():
        engine.step()
    run = engine.runner
    h2d = run._small_len * 4 + batch * run.max_pages * 4 * max(1, len(run.cache.kv_groups))
    return {"value": n / wall, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": batch * 4,
            "ms_per_step": wall * 1000 / steps, "device_ms_per_step": s.elapsed_time(e) / steps}


def run_ours(args):
    import dataclasses
    import torch
    from infurnace_b200.engine import Engine, EngineOptions
    from infurnace_b200.engine.runner import StepEntry
    from infurnace_b200.models import read_config

    hbm_peak, tf_peak, peak_src = read_peaks()
    cfg = read_config(args.config)
    layers_full = cfg.num_hidden_layers
    if args.layers and args.layers < layers_full:
        fields = {"num_hidden_layers": args.layers}
        if getattr(cfg, "layer_types", None) is not None:
            fields["layer_types"] = tuple(cfg.layer_types[:args.layers])
        cfg = dataclasses.replace(cfg, **fields)
    layers_run = cfg.num_hidden_layers
    name = os.path.splitext(os.path.basename(args.config))[0]
    batch, steps, warmup, context = args.batch, args.steps, args.warmup, args.context
    page = args.page_size
    big = max(batch, 64) if args.mode == "all" else batch          # the largest batch of the run
    pool_tokens = big * context + PREFILL_TOKENS + 64
    opts = EngineOptions(dtype="bfloat16", page_size=page, num_pages=pool_tokens // page, max_num_seqs=big,
                         max_num_batched_tokens=PREFILL_TOKENS, max_model_len=context)
    engine = Engine.from_random(cfg, 0, opts)
    runner, plan = engine.runner, engine.plan
    vocab, esize = plan.vocab_size, 2
    if args.eager:
        runner.use_graphs = False
    if args.mode == "prefill":
        times = time_prefill(runner, vocab, max(1, steps), warm=1)
        print(json.dumps({"mode": "prefill", "tokens": PREFILL_TOKENS, "steps": max(1, steps),
                          "ms_median": statistics.median(times), "ms_min": min(times)}))
        return 0
    if args.mode == "generate":
        out = {f"gen_b{b}": time_generation(engine, plan, vocab, b, hbm_peak, esize) for b in sorted({1, batch})}
        print(json.dumps({"mode": "generate", **out}))
        return 0
    randomize_pages(runner)
    torch.cuda.synchronize()
    start_ctx = context - warmup - steps

    # ---- decode, device timed
    clocks = ClockSampler()
    rids = fill_contexts(runner, batch, start_ctx)
    clocks.start()
    ms, launches, per_step = time_decode(runner, rids, vocab, steps, warmup)
    clock_report = clocks.stop()
    release(runner, rids)
    ms_per_step = ms / steps
    value = batch * steps / (ms / 1000.0)
    if args.mode == "decode":
        print(json.dumps({"mode": "decode", "batch": batch, "context": context, "steps": steps, "ms_per_step": ms_per_step,
                          "tokens_per_s": value, "graphs": runner.use_graphs, "launches": launches, "samples": summary(per_step)}))
        return 0
    mean_ctx = context - steps / 2
    w_bytes, kv_bytes = decode_bytes(plan, runner, [mean_ctx] * batch, esize)
    achieved = (w_bytes + kv_bytes) / (ms_per_step / 1000.0) / 1e9

    # ---- decode, end to end through the Engine API (host token ids in and out every step)
    e2e = time_e2e(engine, vocab, batch, context, steps, warmup)

    # ---- prefill of 2,048 tokens in one step
    pre = time_prefill(runner, vocab, 5)
    pre_ms = statistics.median(pre)
    flops = prefill_flops(plan, PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / (pre_ms / 1000.0), "tokens": PREFILL_TOKENS, "ms": pre_ms,
               "frac": flops / (pre_ms / 1000.0) / (tf_peak * 1e12), "tflops": flops / (pre_ms / 1000.0) / 1e12,
               "peak_tflops": tf_peak, "peak_source": peak_src, "min_ms": min(pre), "mean_ms": statistics.fmean(pre)}

    # ---- other batch sizes at the same context
    points, detail = {}, {}
    for b in (1, 64):
        k = max(8, steps // 2)
        rids = fill_contexts(runner, b, context - warmup - k)
        pms, _, ps = time_decode(runner, rids, vocab, k, warmup)
        release(runner, rids)
        points[f"decode_b{b}"] = b * k / (pms / 1000.0)
        wb, kvb = decode_bytes(plan, runner, [context - k / 2] * b, esize)
        s = summary(ps)
        detail[f"decode_b{b}"] = {"us_per_step_min": s["min_ms"] * 1000, "us_per_step_mean": pms / k * 1000,
                                  "us_per_step_median": s["median_ms"] * 1000,
                                  "frac": (wb + kvb) / (pms / k / 1000.0) / 1e9 / hbm_peak}

    # ---- the closed loop of the reference's own benchmark: 128-token prompts, 256 generated tokens
    for b in (1, 8, 64):
        g = time_generation(engine, plan, vocab, b, hbm_peak, esize)
        points[f"gen_b{b}"] = g.pop("tokens_per_s")
        detail[f"gen_b{b}"] = g

    # ---- where the time goes, by class of kernel
    attn_layers = sum(1 for c in plan.resolved_schedule() if getattr(plan.layers[c.layer], "mixer", None) is not None)
    sizes = {"kv_bytes_per_token_per_layer": runner.cache.bytes_per_token() // max(1, attn_layers),
             "attn_flops_per_layer_prefill": (flops - 2 * plan.hidden_size * vocab
                                              - sum(2 * s.shape[0] * s.shape[1] * PREFILL_TOKENS
                                                    for c in plan.resolved_schedule()
                                                    for s in plan.layers[c.layer].tensors().values() if len(s.shape) == 2))
             // max(1, attn_layers)}
    kernels = profile_classes(runner, plan, sizes, batch, context, vocab, esize)

    def rounded(d):
        return {k: (round(v, 4) if isinstance(v, float) else v) for k, v in d.items()}

    mixer = plan.layers[0].mixer
    ffn = plan.layers[0].ffn
    line = {
        "metric": f"decode tok/s at batch {batch}, context {context} ({name} shape, random weights)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"model": f"{name} shape, random weights drawn on the device, seed 0", "layers": layers_full,
                   "layers_run": layers_run, "hidden": plan.hidden_size, "heads": mixer.num_heads,
                   "kv_heads": mixer.num_kv_heads, "head_dim": mixer.head_dim, "intermediate": ffn.intermediate_size,
                   "vocab": vocab, "global_batch": batch, "seq_len": context, "page_size": page,
                   "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU",
                   "l2": f"inputs larger than L2 (weights {w_bytes / 1e9:.1f} GB + KV {kv_bytes / 1e9:.1f} GB)",
                   "context_fill": "random keys/values in pages"},
        "samples": rounded(summary(per_step)),
        "e2e": e2e, "gpu_launches": launches, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "bytes_per_step": w_bytes + kv_bytes, "peak_source": peak_src},
        "points": points, "points_detail": {k: rounded(v) for k, v in detail.items()}, "kernels": kernels,
        "clocks": clock_report,
    }
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096, help="tokens each request holds in the timed decode steps")
    ap.add_argument("--config", default=os.path.join(ROOT, "configs", "qwen3-0.6b.json"),
                    help="config.json of the model whose sizes are run (random weights)")
    ap.add_argument("--layers", type=int, default=0, help="run only this many layers (0: all the configuration has)")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per page of the key/value cache")
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--mode", default="all", choices=("all", "decode", "prefill", "generate"),
                    help="decode / prefill / generate: only that part, on a pool just large enough (for profiling a small case)")
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
