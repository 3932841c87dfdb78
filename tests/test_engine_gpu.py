"""Generation through the entry points on the GPU: greedy and temperature sampling against the
plain implementation, decode steps replayed from CUDA graphs, preemption, and the command line."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen3 as P
import tiny
from infurnace_b200.engine import Engine, EngineOptions, Request, RequestState, SamplingParams, generate
from infurnace_b200.sampling import uniform

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("models"))
    return {n: tiny.make_model_dir(n, root) for n in tiny.TINY}


def engine(model_dir, name, dtype, **kw):
    opts = dict(dtype=dtype, page_size=tiny.TINY[name]["page_size"], num_pages=64, max_num_seqs=4,
                max_num_batched_tokens=64)
    opts.update(kw)
    return Engine.from_model_dir(model_dir, EngineOptions(**opts))


def near_top(cfg, w, prompt, tokens, margin):
    """Every generated token is, given its own prefix, within ``margin`` of the plain top logit."""
    seq = list(prompt)
    for t in tokens:
        logits = P.forward(cfg, w, seq)[-1]
        assert float(logits.max() - logits[t]) <= margin, (len(seq), t, int(logits.argmax()))
        seq.append(t)


@pytest.mark.parametrize("name", list(tiny.TINY))
def test_greedy_float32_equals_the_plain_implementation(models, name):
    cfg, w = P.read_model(models[name])
    eng = engine(models[name], name, "float32")
    prompts = [tiny.random_tokens(cfg["vocab_size"], n, 50 + n) for n in (1, 7, 33)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=16))
    for p, o in zip(prompts, outs):
        want = P.greedy(cfg, w, p, 16)
        if o != want:
            near_top(cfg, w, p, o, 1e-5)       # only an exact tie in float32 may part them
    assert eng.runner.graph_replays > 0          # decode steps came from graphs
    eng.runner.cache.check()


@pytest.mark.parametrize("name", list(tiny.TINY))
def test_greedy_bfloat16_stays_at_the_top(models, name):
    cfg, w = P.read_model(models[name])
    eng = engine(models[name], name, "bfloat16")
    prompts = [tiny.random_tokens(cfg["vocab_size"], n, 60 + n) for n in (1, 7, 33, 100)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=16))
    for p, o in zip(prompts, outs):
        assert len(o) == 16
        near_top(cfg, w, p, o, 0.05)
    assert eng.runner.graph_replays > 0


def test_graph_replay_equals_eager_steps(models):
    a = engine(models["B"], "B", "bfloat16")
    b = engine(models["B"], "B", "bfloat16")
    b.runner.use_graphs = False
    prompts = [tiny.random_tokens(320, n, 70 + n) for n in (5, 19, 64)]
    sp = SamplingParams(max_tokens=40, temperature=0.7, seed=3)
    assert a.generate(prompts, sp) == b.generate(prompts, sp)
    assert a.runner.graph_replays > 0 and b.runner.graph_replays == 0


def test_temperature_sampling_follows_the_requests_own_numbers(models):
    cfg, w = P.read_model(models["B"])
    prompts = [tiny.random_tokens(320, n, 20 + n) for n in (5, 19, 64, 100)]
    sps = [SamplingParams(max_tokens=12, temperature=0.8, seed=100 + i) for i in range(4)]
    eng = engine(models["B"], "B", "float32", max_num_batched_tokens=16)      # portions of 16 beside decode tokens
    together = eng.generate(prompts, sps)
    alone = [engine(models["B"], "B", "float32", max_num_batched_tokens=256).generate([p], sp)[0]
             for p, sp in zip(prompts, sps)]
    assert together == alone
    for p, sp, out in zip(prompts, sps, together):
        seq = list(p)
        for k, t in enumerate(out):
            probs = P.temperature_probs(P.forward(cfg, w, seq)[-1], 0.8).double().cumsum(0)
            u = uniform(sp.seed, k)
            want = int(torch.searchsorted(probs, torch.tensor(u, dtype=torch.float64), right=True))
            if t != want:     # u may sit on a boundary of the running sum
                assert abs(t - want) == 1 and min(abs(float(probs[t]) - u), abs(float(probs[want]) - u)) < 1e-4
            seq.append(t)


def test_preemption_round_trip_on_the_gpu(models):
    cfg, w = P.read_model(models["A"])
    prompts = [tiny.random_tokens(256, n, 30 + n) for n in (30, 28, 25)]
    small = engine(models["A"], "A", "float32", num_pages=6)
    outs = small.generate(prompts, SamplingParams(max_tokens=30))
    assert small.scheduler.num_preemptions > 0
    roomy = engine(models["A"], "A", "float32").generate(prompts, SamplingParams(max_tokens=30))
    assert outs == roomy
    small.runner.cache.check()
    assert small.runner.cache.free_pages() == [6]


def test_tool_style_entry_point_and_command_line(models, tmp_path):
    eng = engine(models["A"], "A", "bfloat16")
    toks, timings = generate(eng, [5, 6, 7], 4)
    assert len(toks) == 7 and timings["prefill_ms"] > 0 and len(timings["decode_times_ms"]) == 3
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bin", "infurnace-b200"), "--model", models["A"],
                          "--prompt-ids", "5,6,7", "--max-tokens", "4", "--json", "--page-size", "16",
                          "--max-context", "64"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    report = json.loads(out.stdout)
    assert report["prompt"] == [5, 6, 7] and report["generated_token_ids"] == toks[3:]
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(tiny.TINY["B"]["config"]))
    out = subprocess.run([sys.executable, "-m", "infurnace_b200", "--random-weights", "3", "--config", str(cfg_path),
                          "--prompt", "hello", "--char-tokenizer", "--max-tokens", "5", "--page-size", "8",
                          "--max-context", "64", "--temperature", "0.9", "--seed", "4"],
                         capture_output=True, text=True, timeout=300, cwd=root)
    assert out.returncode == 0, out.stderr
    assert len(out.stdout.rstrip("\n")) == 5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_launching_ahead_changes_no_token_on_the_gpu(models, dtype):
    """Graph-replayed decode steps launched before the previous step's tokens are read, against the
    one-step-at-a-time loop: stop tokens cut requests short, lengths differ, requests outnumber slots."""
    prompts = [tiny.random_tokens(320, n, 40 + n) for n in (5, 19, 33, 8, 50, 3)]
    base = engine(models["B"], "B", dtype, max_num_seqs=3)
    base.overlap_decode = False
    free_run = base.generate(prompts, SamplingParams(max_tokens=20, temperature=0.9, seed=5))
    stops = sorted({t[7] for t in free_run} | {free_run[0][2]})
    sps = [SamplingParams(max_tokens=10 + 3 * i, temperature=0.9, seed=5, stop_token_ids=stops, min_tokens=i % 3)
           for i in range(len(prompts))]
    outs = {}
    for overlap in (False, True):
        eng = engine(models["B"], "B", dtype, max_num_seqs=3)
        eng.overlap_decode = overlap
        outs[overlap] = eng.generate(prompts, sps)
        eng.runner.cache.check()
        assert eng.is_done() and eng.runner.graph_replays > 0
    assert outs[True] == outs[False]
    assert any(len(o) < sp.max_tokens for o, sp in zip(outs[True], sps))


def test_a_fault_recorded_in_the_error_word_fails_the_requests_that_ran(models):
    """The device error word set between steps (written from the host here; no kernel is made to give up): the
    requests that ran since it was last read clean end FAILED with their pages and slots back, none of them is
    reported finished, and the engine serves the next request."""
    eng = engine(models["B"], "B", "bfloat16")
    eng.add_request(Request("long", tiny.random_tokens(320, 9, 1), SamplingParams(max_tokens=50)))
    eng.add_request(Request("short", tiny.random_tokens(320, 5, 2), SamplingParams(max_tokens=3)))
    eng.step()
    K = eng.runner.rt.kernels
    torch.cuda.synchronize()
    K._dev_err.fill_(7)
    failed, completed = [], []
    for _ in range(10):
        res = eng.step()
        failed += list(res.failed_requests)
        completed += list(res.completed_requests)
        if eng.is_done():
            break
    assert sorted(failed) == ["long", "short"] and not completed
    for rid in ("long", "short"):
        r = eng.scheduler.get_request(rid)
        assert r.state is RequestState.FAILED and "code 7" in r.error
    assert eng.is_done() and eng.runner.cache.free_pages() == [64, 64]
    eng.runner.cache.check()
    assert len(eng.generate([tiny.random_tokens(320, 4, 3)], SamplingParams(max_tokens=4))[0]) == 4


def test_sampler_for_callers_that_hold_logits_draws_what_the_engine_draws(models):
    """``Sampler`` on the logits of ``ModelRunner.step`` gives the token the engine samples inside its
    step: the same kernel and the same (seed, counter) numbers."""
    from infurnace_b200.engine.runner import StepEntry
    from infurnace_b200.sampling import Sampler
    prompt = tiny.random_tokens(320, 21, 9)
    sp = SamplingParams(max_tokens=6, temperature=0.8, seed=77)
    want = engine(models["B"], "B", "float32").generate([prompt], sp)[0]
    eng = engine(models["B"], "B", "float32")
    run = eng.runner
    sampler = Sampler(run.rt.kernels, run.rt.device)
    run.cache.add_request("x")
    toks, got = list(prompt), []
    for k in range(6):
        logits = run.step([StepEntry("x", toks, [len(toks) - 1])])
        got += sampler.sample(logits, [0.8], [77], [k])
        toks = [got[-1]]
    assert got == want
    assert sampler.sample(logits, [0.0], [0], [0]) == [int(logits[0].argmax())]


def test_random_weights_drawn_on_the_device_equal_the_folders(tmp_path):
    """``Engine.from_random`` without a folder (tensors drawn by the kernel as the parts ask for them) against
    the folder writer on the host followed by the loader: the same fused matrices, the same tokens."""
    from infurnace_b200.models import config_from_dict
    cfg = config_from_dict(tiny.TINY["C"]["config"])
    opts = dict(dtype="bfloat16", page_size=32, num_pages=16, max_num_seqs=2, max_num_batched_tokens=64)
    a = Engine.from_random(cfg, 4, EngineOptions(**opts))
    b = Engine.from_random(cfg, 4, EngineOptions(**opts), workdir=str(tmp_path / "m"))
    for la, lb in zip(a.runner.model.layers, b.runner.model.layers):
        assert torch.equal(la.mixer.w_qkv, lb.mixer.w_qkv) and torch.equal(la.ffn.w_gate_up, lb.ffn.w_gate_up)
        assert torch.equal(la.mixer_norm.weight, lb.mixer_norm.weight)
    assert a.runner.model.lm_head.weight.data_ptr() == a.runner.model.embedding.table.data_ptr()      # tied: one tensor
    prompt = tiny.random_tokens(333, 12, 1)
    assert a.generate([prompt], SamplingParams(max_tokens=8)) == b.generate([prompt], SamplingParams(max_tokens=8))
