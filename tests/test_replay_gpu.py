"""The engine against the plain implementation, every way of cutting the work, in float32 and
in bfloat16: whole requests; most of a request in one step and its last 32 tokens one by one;
portions of changing size down to two tokens; and up to four live requests mixed, portions of
some beside decoded tokens of others, in a pool so small that pages are used again."""
import os

import pytest
import torch

import plain_qwen3 as P
import tiny

pytestmark = pytest.mark.gpu

LENS = [37, 100, 64, 19, 85, 50, 1, 2, 128]
# float32: the engine and the plain implementation differ by rounding only
F32_TOL = 2e-5
# bfloat16: activations between kernels carry 8 bits of mantissa; logits here are of size 1
BF16_TOL = 4e-2


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("models"))
    out = {}
    for name in tiny.TINY:
        d = tiny.make_model_dir(name, root)
        cfg, w = P.read_model(d)
        limit = cfg["max_position_embeddings"]
        reqs = {f"r{i}": tiny.random_tokens(cfg["vocab_size"], min(n, limit), 100 + i) for i, n in enumerate(LENS)}
        ref = {r: P.forward(cfg, w, t) for r, t in reqs.items()}
        out[name] = (d, cfg, reqs, ref)
    return out


def _runner(model_dir, name, dtype, pool_tokens, max_seqs=4):
    from infurnace_b200.engine.loading import EngineOptions, build_runner
    ps = tiny.TINY[name]["page_size"]
    opts = EngineOptions(dtype=dtype, device="cuda", page_size=ps, num_pages=pool_tokens // ps, max_num_seqs=max_seqs,
                         max_num_batched_tokens=pool_tokens)
    return build_runner(model_dir, opts)[2]


def _schedules(reqs):
    return {
        "whole": tiny.schedule_whole(reqs),
        "bulk_tail": tiny.schedule_bulk_tail(reqs, tail=32),
        "portions": tiny.schedule_portions(reqs, seed=1),
        "mixed": tiny.schedule_mixed(reqs, max_live=4, max_tokens=320, seed=2),
    }


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "bulk_tail", "portions", "mixed"])
@pytest.mark.parametrize("name", list(tiny.TINY))
def test_cutting_modes(models, name, mode, dtype):
    d, cfg, reqs, ref = models[name]
    steps = _schedules(reqs)[mode]
    runner = _runner(d, name, dtype, 320)
    out = tiny.collect(steps, tiny.run_inprocess(runner, steps), cfg["vocab_size"])
    assert all(p == runner.cache.kv_groups[i].pool.num_pages for i, p in enumerate(runner.cache.free_pages()))
    tolerance = F32_TOL if dtype == "float32" else BF16_TOL
    worst = ("", 0, 0.0)
    for rid in reqs:
        err = (out[rid] - ref[rid]).abs().max(dim=-1).values
        pos = int(err.argmax())
        if float(err[pos]) > worst[2]:
            worst = (rid, pos, float(err[pos]))
    assert worst[2] <= tolerance, f"{name} {mode} {dtype}: first look at request {worst[0]} position {worst[1]}: {worst[2]}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decode(models, dtype):
    """The first tokens of a sequence one by one, then decoding on to the model's limit."""
    d, cfg, reqs, ref = models["B"]
    toks = tiny.random_tokens(cfg["vocab_size"], cfg["max_position_embeddings"], 7)
    want = P.forward(cfg, P.read_model(d)[1], toks)
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
    runner = _runner(d, "B", dtype, 256)
    out = tiny.collect(steps, tiny.run_inprocess(runner, steps), cfg["vocab_size"])["x"]
    err = (out - want).abs().max(dim=-1).values
    tolerance = F32_TOL if dtype == "float32" else BF16_TOL
    assert float(err.max()) <= tolerance, f"position {int(err.argmax())}: {float(err.max())}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(models, tmp_path, dtype):
    """bin/trace_run as a child process, mixed schedule, files on disk."""
    d, cfg, reqs, ref = models["A"]
    steps = tiny.schedule_mixed(reqs, max_live=4, max_tokens=320, seed=5)
    outputs = tiny.run_trace_run(d, dtype, steps, str(tmp_path / "out"), 320, tiny.TINY["A"]["page_size"])
    out = tiny.collect(steps, outputs, cfg["vocab_size"])
    tolerance = F32_TOL if dtype == "float32" else BF16_TOL
    for rid in reqs:
        assert float((out[rid] - ref[rid]).abs().max()) <= tolerance
