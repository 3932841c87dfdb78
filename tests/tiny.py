"""Tiny configurations of the architecture, model folders made from them, and the
schedules (ways of cutting requests into steps) that the replay tests run."""
from __future__ import annotations

import json
import os
import random

import torch

QWEN3 = "Qwen3ForCausalLM"

# Configurations that differ in every size and option.
TINY = {
    # 2 layers, every key visible, tied head, float32 storage
    "A": dict(config=dict(architectures=[QWEN3], num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
                          num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256,
                          rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                          max_position_embeddings=128),
              page_size=16, store_dtype="float32", seed=11),
    # 3 layers, group ratio 4, q width != hidden, untied head, a window on the middle layer, bfloat16 storage
    "B": dict(config=dict(architectures=[QWEN3], num_hidden_layers=3, hidden_size=96, num_attention_heads=8,
                          num_key_value_heads=2, head_dim=32, intermediate_size=160, vocab_size=320,
                          rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
                          max_position_embeddings=256, sliding_window=24,
                          layer_types=["full_attention", "sliding_attention", "full_attention"]),
              page_size=8, store_dtype="bfloat16", seed=22),
    # the same sizes without any window
    "B0": dict(config=dict(architectures=[QWEN3], num_hidden_layers=3, hidden_size=96, num_attention_heads=8,
                           num_key_value_heads=2, head_dim=32, intermediate_size=160, vocab_size=320,
                           rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
                           max_position_embeddings=256),
               page_size=8, store_dtype="float32", seed=22),
    # nothing is a power of two: 6 heads in 3 groups of head size 48, widths 72/136, vocabulary 333,
    # windows on the first and last layer, norm weights stored in float32 beside bfloat16 matrices
    "C": dict(config=dict(architectures=[QWEN3], num_hidden_layers=4, hidden_size=72, num_attention_heads=6,
                          num_key_value_heads=3, head_dim=48, intermediate_size=136, vocab_size=333,
                          rope_theta=500000.0, rms_norm_eps=3e-6, tie_word_embeddings=True,
                          max_position_embeddings=192, sliding_window=40,
                          layer_types=["sliding_attention", "full_attention", "full_attention", "sliding_attention"]),
              page_size=32, store_dtype="bfloat16", norm_dtype="float32", seed=33),
}


def make_model_dir(name: str, root: str, sharpen: float = 3.0) -> str:
    """Write tiny model ``name`` under ``root``.  The q_norm weights are scaled by ``sharpen``,
    which makes the attention scores spread (standard deviation about ``sharpen``) so that a
    wrong, missing or stale key changes the logits visibly."""
    from infurnace_b200.models import config_from_dict
    from infurnace_b200.weights.random_init import write_random_model
    from safetensors.torch import load_file, save_file
    spec = TINY[name]
    cfg = config_from_dict(spec["config"])
    d = os.path.join(root, f"tiny{name}")
    write_random_model(cfg, spec["seed"], d, store_dtype=spec["store_dtype"], norm_dtype=spec.get("norm_dtype"))
    if sharpen != 1.0:
        path = os.path.join(d, "model.safetensors")
        tensors = load_file(path)
        for k in list(tensors):
            if k.endswith("q_norm.weight"):
                tensors[k] = (tensors[k].float() * sharpen).to(tensors[k].dtype)
        save_file(tensors, path)
    return d


def random_tokens(vocab: int, n: int, seed: int):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


# ------------------------------------------------------------------------------ schedules
def _entry(rid, toks, start, n):
    return {"id": rid, "tokens": toks[start:start + n], "want": list(range(n))}


def schedule_whole(requests):
    """Each request alone, its whole sequence in one step."""
    return [{"step": i, "entries": [_entry(rid, toks, 0, len(toks))], "end": [rid]}
            for i, (rid, toks) in enumerate(requests.items())]


def schedule_bulk_tail(requests, tail=32):
    """All but the last ``tail`` tokens in one step, then one token per step."""
    steps = []
    for rid, toks in requests.items():
        cut = max(1, len(toks) - tail)
        cuts = [(0, cut)] + [(i, 1) for i in range(cut, len(toks))]
        for j, (s, n) in enumerate(cuts):
            steps.append({"step": len(steps), "entries": [_entry(rid, toks, s, n)],
                          "end": [rid] if j == len(cuts) - 1 else []})
    return steps


def schedule_portions(requests, seed=0):
    """Each request alone in portions of changing size, down to two tokens."""
    rng = random.Random(seed)
    sizes = [7, 2, 16, 3, 2, 33, 5, 2, 9, 17, 2, 31]
    steps = []
    for rid, toks in requests.items():
        s = 0
        while s < len(toks):
            n = min(len(toks) - s, rng.choice(sizes))
            steps.append({"step": len(steps), "entries": [_entry(rid, toks, s, n)],
                          "end": [rid] if s + n == len(toks) else []})
            s += n
    return steps


def schedule_mixed(requests, max_live=4, max_tokens=256, tail=12, seed=0, unit=64, sizes=(2, 3, 5, 8, 13, 16, 21)):
    """Up to ``max_live`` requests at a time: portions of some (of the ``sizes``) beside single
    decoded tokens of others, a request sometimes left out of a step, under a pool of
    ``max_tokens`` tokens (each live request counted rounded up to ``unit``), so that pages are
    used again."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live = {}      # rid -> progress
    steps = []

    def held():
        return sum(-(-len(requests[r]) // unit) * unit for r in live)

    while waiting or live:
        while waiting and len(live) < max_live and held() + -(-len(waiting[0][1]) // unit) * unit <= max_tokens:
            rid, _ = waiting.pop(0)
            live[rid] = 0
        if not live:
            raise ValueError("max_tokens is too small for the first waiting request")
        entries, ended = [], []
        chosen = [r for r in live if rng.random() < 0.8] or [next(iter(live))]
        for rid in chosen:
            toks, s = requests[rid], live[rid]
            left = len(toks) - s
            n = 1 if left <= tail else min(left - tail, rng.choice(list(sizes)))
            entries.append(_entry(rid, toks, s, n))
            live[rid] = s + n
            if s + n == len(toks):
                ended.append(rid)
        for rid in ended:
            del live[rid]
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def collect(steps, outputs, vocab):
    """Per request, the logits of every position in order.  ``outputs``: step -> [wanted, vocab]."""
    per = {}
    for st in steps:
        out = outputs.get(st["step"])
        row = 0
        for e in st["entries"]:
            for _ in e["want"]:
                per.setdefault(e["id"], []).append(out[row])
                row += 1
        assert out is None or row == out.shape[0]
    return {rid: torch.stack(rows) for rid, rows in per.items()}


def run_inprocess(runner, steps):
    """Drive ``runner`` (the engine's step function) through ``steps``."""
    from infurnace_b200.engine.runner import StepEntry
    outputs = {}
    for st in steps:
        entries = []
        for e in st["entries"]:
            if not runner.cache.has_request(e["id"]):
                runner.cache.add_request(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        logits = runner.step(entries)
        if logits is not None:
            outputs[st["step"]] = logits.float().cpu().clone()
        for rid in st["end"]:
            runner.cache.free_request(rid)
        runner.cache.check()
    return outputs


def run_trace_run(model_dir, dtype, steps, out_dir, max_tokens, page_size, env=None):
    """Drive ``bin/trace_run`` as a child process through ``steps``."""
    import subprocess
    import sys
    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens), "--page-size", str(page_size)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    for st in steps:
        proc.stdin.write(json.dumps(st) + "\n")
        proc.stdin.flush()
        line = proc.stdout.readline().strip()
        assert line == f"done {st['step']}", f"trace_run answered {line!r}"
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0
    outputs = {}
    for st in steps:
        path = os.path.join(out_dir, f"{st['step']}.f32")
        wanted = sum(len(e["want"]) for e in st["entries"])
        if wanted:
            data = np.fromfile(path, dtype="<f4")
            outputs[st["step"]] = torch.from_numpy(data.reshape(wanted, -1).copy())
    return outputs
