"""The host side of the engine on a machine without a GPU: the step function, the scheduler and
the engine loop run over the plain kernel statements of tests/kernel_refs.py in place of the
CUDA kernels, and are compared with the plain implementation.  (The package itself never runs
this way: its kernel set needs a CUDA device.)"""
import io
import sys

import pytest
import torch

import plain_qwen3 as P
import tiny
from kernel_refs import ReferenceKernels
from infurnace_b200.engine import Engine, EngineOptions, Request, RequestState, SamplingParams, StepEntry, generate
from infurnace_b200.errors import BatchError, KernelError, OutOfPages


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("models"))
    return {n: tiny.make_model_dir(n, root) for n in tiny.TINY}


def engine(model_dir, name, **kw):
    opts = dict(dtype="float32", device="cpu", page_size=tiny.TINY[name]["page_size"], num_pages=40, max_num_seqs=4,
                max_num_batched_tokens=64)
    opts.update(kw)
    return Engine.from_model_dir(model_dir, EngineOptions(**opts), kernels=ReferenceKernels())


@pytest.mark.parametrize("name", list(tiny.TINY))
@pytest.mark.parametrize("mode", ["whole", "bulk_tail", "portions", "mixed"])
def test_cutting_modes_on_the_host_path(models, name, mode):
    cfg, w = P.read_model(models[name])
    lens = [37, 100, 64, 19, 85, 50, 1, 2]
    reqs = {f"r{i}": tiny.random_tokens(cfg["vocab_size"], n, i) for i, n in enumerate(lens)}
    steps = {"whole": tiny.schedule_whole, "bulk_tail": tiny.schedule_bulk_tail, "portions": tiny.schedule_portions,
             "mixed": lambda r: tiny.schedule_mixed(r, max_tokens=320)}[mode](reqs)
    eng = engine(models[name], name, num_pages=320 // tiny.TINY[name]["page_size"], max_num_batched_tokens=320)
    out = tiny.collect(steps, tiny.run_inprocess(eng.runner, steps), cfg["vocab_size"])
    for rid, toks in reqs.items():
        assert (out[rid] - P.forward(cfg, w, toks)).abs().max() < 2e-5, (rid, mode)


def test_a_norm_folded_into_its_neighbours_changes_no_logit(models):
    """Steps of few tokens leave the norms between products to the products (the one before
    writes x * weight and partial sums of squares, the one after applies the rows' factors);
    steps of many tokens run the norm's own kernel.  Both give the plain implementation's logits,
    also where a small step follows a large one and where a layer is the last."""
    cfg, w = P.read_model(models["B"])
    toks = tiny.random_tokens(cfg["vocab_size"], 120, 5)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:90], "want": [0, 89]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[90:118], "want": [0, 27]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[118:], "want": [0, 1]}], "end": ["a"]}]
    ref = P.forward(cfg, w, toks)
    calls = {}
    for fold in (True, False):
        kernels = ReferenceKernels(fold=fold)
        count = [0]
        inner = kernels.linear_residual_norm

        def spy(*a, _inner=inner, _count=count, **kw):
            _count[0] += 1
            return _inner(*a, **kw)
        kernels.linear_residual_norm = spy
        opts = EngineOptions(dtype="float32", device="cpu", page_size=tiny.TINY["B"]["page_size"], num_pages=40,
                             max_num_seqs=4, max_num_batched_tokens=128)
        eng = Engine.from_model_dir(models["B"], opts, kernels=kernels)
        out = tiny.collect(steps, tiny.run_inprocess(eng.runner, steps), cfg["vocab_size"])
        rows = [0, 89, 90, 117, 118, 119]
        assert (out["a"] - ref[rows]).abs().max() < 2e-5, fold
        calls[fold] = count[0]
    layers = cfg["num_hidden_layers"]
    assert calls[False] == 0
    assert calls[True] == 2 * (2 * layers - 1)      # two small steps; every norm but the first of a step and the final one


def test_greedy_generation_equals_the_plain_implementation(models):
    cfg, w = P.read_model(models["A"])
    eng = engine(models["A"], "A")
    prompts = [tiny.random_tokens(256, n, 10 + n) for n in (1, 7, 33)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=16))
    for p, o in zip(prompts, outs):
        assert o == P.greedy(cfg, w, p, 16)
    eng.runner.cache.check()
    assert eng.runner.cache.free_pages() == [40]


def test_temperature_sampling_does_not_depend_on_batching_or_portions(models):
    eng = engine(models["B"], "B", max_num_batched_tokens=16)        # portions of 16 beside decode tokens
    prompts = [tiny.random_tokens(320, n, 20 + n) for n in (5, 19, 64, 100)]
    sps = [SamplingParams(max_tokens=12, temperature=0.8, seed=100 + i) for i in range(4)]
    together = eng.generate(prompts, sps)
    alone = [engine(models["B"], "B", max_num_batched_tokens=256).generate([p], sp)[0] for p, sp in zip(prompts, sps)]
    assert together == alone
    assert len({tuple(t) for t in together}) == 4
    other_seed = engine(models["B"], "B").generate([prompts[1]], SamplingParams(max_tokens=12, temperature=0.8, seed=7))[0]
    assert other_seed != together[1]
    # the drawn token is the inverse CDF of the request's own uniform number
    from infurnace_b200.sampling import uniform
    cfg, w = P.read_model(models["B"])
    probs = P.temperature_probs(P.forward(cfg, w, prompts[0])[-1], 0.8).double().cumsum(0)
    u = uniform(100, 0)
    assert together[0][0] == int(torch.searchsorted(probs, torch.tensor(u, dtype=torch.float64), right=True))


def test_preemption_round_trip_gives_the_same_tokens(models):
    cfg, w = P.read_model(models["A"])
    prompts = [tiny.random_tokens(256, n, 30 + n) for n in (30, 28, 25)]
    small = engine(models["A"], "A", num_pages=6, max_num_batched_tokens=64)      # 96 tokens of pool for 3 x 60
    outs = small.generate(prompts, SamplingParams(max_tokens=30))
    assert small.scheduler.num_preemptions > 0
    for p, o in zip(prompts, outs):
        assert o == P.greedy(cfg, w, p, 30)
    small.runner.cache.check()
    assert small.runner.cache.free_pages() == [6]


def test_out_of_pages_fails_the_lone_request_and_frees_everything(models):
    eng = engine(models["A"], "A", num_pages=2)
    eng.add_request(Request("big", tiny.random_tokens(256, 30, 1), SamplingParams(max_tokens=40)))
    for _ in range(50):
        if eng.is_done():
            break
        eng.step()
    r = eng.scheduler.get_request("big")
    assert r.state is RequestState.FAILED and r.error == "out of KV pages" and len(r.output_token_ids) == 3
    assert eng.runner.cache.free_pages() == [2]


def test_a_failing_step_fails_its_requests_and_the_engine_goes_on(models, monkeypatch, capsys):
    eng = engine(models["A"], "A")
    eng.add_request(Request("a", [1, 2, 3], SamplingParams(max_tokens=4)))
    real = eng.runner.step_and_sample
    monkeypatch.setattr(eng.runner, "step_and_sample",
                        lambda *a, **kw: (_ for _ in ()).throw(RuntimeError("device fell over")))
    res = eng.step()
    assert res.failed_requests == ("a",)
    a = eng.scheduler.get_request("a")
    assert a.state is RequestState.FAILED and "device fell over" in a.error
    assert eng.runner.cache.free_pages() == [40] and eng.is_done()
    monkeypatch.setattr(eng.runner, "step_and_sample", real)
    assert len(eng.generate([[4, 5, 6]], SamplingParams(max_tokens=3))[0]) == 3


@pytest.mark.parametrize("temperature", [0.0, 0.9])
def test_launching_ahead_changes_no_token(models, temperature):
    """Decode steps launched before the previous step's tokens are read (input tokens taken on the
    device) give the tokens of the plain one-step-at-a-time loop: with stop tokens that cut requests
    short (the token computed too many is dropped), different lengths, and more requests than slots."""
    cfg, w = P.read_model(models["B"])
    prompts = [tiny.random_tokens(320, n, 40 + n) for n in (5, 19, 33, 8, 50, 3)]
    base = engine(models["B"], "B", max_num_seqs=3)
    base.overlap_decode = False
    free_run = base.generate(prompts, SamplingParams(max_tokens=20, temperature=temperature, seed=5))
    stops = sorted({t[7] for t in free_run} | {free_run[0][2]})       # tokens that really occur: requests stop early
    sps = [SamplingParams(max_tokens=10 + 3 * i, temperature=temperature, seed=5, stop_token_ids=stops, min_tokens=i % 3)
           for i in range(len(prompts))]
    outs = {}
    for overlap in (False, True):
        eng = engine(models["B"], "B", max_num_seqs=3)
        eng.overlap_decode = overlap
        outs[overlap] = eng.generate(prompts, sps)
        eng.runner.cache.check()
        assert eng.runner.cache.free_pages() == [40, 40] and eng.is_done()
    assert outs[True] == outs[False]
    assert any(len(o) < sp.max_tokens for o, sp in zip(outs[True], sps))       # some did stop on a stop token


def test_cancel_between_steps(models):
    eng = engine(models["A"], "A")
    eng.add_request(Request("a", [1, 2, 3], SamplingParams(max_tokens=50)))
    eng.add_request(Request("b", [4, 5], SamplingParams(max_tokens=5)))
    eng.step()
    eng.step()
    eng.cancel("a")
    n = len(eng.output_tokens("a"))
    while not eng.is_done():
        eng.step()
    assert len(eng.output_tokens("a")) == n and eng.scheduler.get_request("a").state is RequestState.CANCELLED
    assert len(eng.output_tokens("b")) == 5 and eng.runner.cache.free_pages() == [40]


def test_step_function_refuses_malformed_batches(models):
    eng = engine(models["A"], "A", num_pages=4, max_num_batched_tokens=32)
    run, cache = eng.runner, eng.runner.cache
    cache.add_request("a")
    for bad, what in [([], "at least one"), ([StepEntry("zz", [1])], "not live"), ([StepEntry("a", [])], "no tokens"),
                      ([StepEntry("a", [256])], "vocabulary"), ([StepEntry("a", [1, 2], [2])], "place 2"),
                      ([StepEntry("a", [1]), StepEntry("a", [2])], "twice"), ([StepEntry("a", [1] * 33)], "at most 32")]:
        with pytest.raises(BatchError, match=what):
            run.step(bad)
    cache.add_request("b")
    with pytest.raises(OutOfPages):
        run.step([StepEntry("a", [1] * 20), StepEntry("b", [1] * 12), ])   # fits the budget...
        run.step([StepEntry("a", [1] * 30), StepEntry("b", [1] * 2)])      # ...but 5 pages are needed
    cache.check()
    assert cache.num_computed("a") in (0, 20)


def test_text_requests_stop_strings_and_the_tool_style_entry_point(models):
    from infurnace_b200.tokenizer import CharTokenizer
    opts = EngineOptions(dtype="float32", device="cpu", page_size=16, num_pages=40, max_num_seqs=2, max_num_batched_tokens=64)
    eng = Engine.from_model_dir(models["A"], opts, tokenizer=CharTokenizer(256), kernels=ReferenceKernels())
    req = eng.add_text_request("hello", SamplingParams(max_tokens=12))
    text = ""
    while not eng.is_done():
        text += "".join(eng.step().new_text.values())
    assert text == eng.final_text(req.request_id) and len(text) == 12
    stop = text[4:6]
    req2 = eng.add_text_request("hello", SamplingParams(max_tokens=12), stop_strings=[stop])
    while not eng.is_done():
        eng.step()
    assert eng.final_text(req2.request_id) == text[:text.find(stop)]
    assert eng.scheduler.get_request(req2.request_id).finish_reason == "stop"
    assert eng.metrics_of(req2.request_id).ttft is not None
    toks, timings = generate(eng, [5, 6, 7], 4)
    assert len(toks) == 7 and {"prefill_ms", "first_decode_ms", "avg_decode_ms", "decode_times_ms"} <= set(timings)


def test_command_line_argument_errors(capsys):
    from infurnace_b200.cli import main
    assert main(["--prompt-ids", "1,2", "--model", "/nonexistent"]) == 1
    assert "not found" in capsys.readouterr().err
    assert main(["--prompt-ids", "1,2"]) == 1
    assert main(["--prompt-ids", "1", "--prompt-len", "3", "--model", "x"]) == 1
    assert main(["--prompt-ids", "1", "--model", "x", "--device", "cpu"]) == 1
    assert "no CPU path" in capsys.readouterr().err


def test_the_package_has_no_cpu_path():
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from infurnace_b200.kernels import load_cuda_kernels
    with pytest.raises(KernelError, match="no CUDA device"):
        load_cuda_kernels()


def test_decode_padding_fits_the_staging_regions_when_slots_exceed_the_token_budget(models):
    """A decode-only step is padded to a power-of-two number of requests.  With a token budget smaller
    than that (3 tokens a step, 4 slots, 3 decoders) the padded step has more rows than max_tokens: the
    staging regions are sized for it, no region runs into its neighbour, and every pad row stores nowhere."""
    eng = engine(models["B"], "B", max_num_batched_tokens=3, max_num_seqs=4)
    run, cache = eng.runner, eng.runner.cache
    for rid in "abc":
        cache.add_request(rid)
        run.step([StepEntry(rid, [1, 2, 3])])
    entries = [StepEntry(rid, [5], [0]) for rid in "abc"]
    run.validate(entries, sampled=True)
    run._reserve(entries)
    ctx = run._build_context(entries, temperatures=[0.7] * 3, uniforms=[0.5] * 3, pad_to=4, seq_bucket=256)
    assert ctx.num_tokens == 4 and ctx.num_requests == 4
    for gi in range(len(cache.kv_groups)):
        slots = ctx.group_slot_mapping[gi].tolist()
        assert slots[3] == -1 and all(s >= 0 for s in slots[:3])
    assert ctx.positions.tolist() == [3, 3, 3, 0] and ctx.token_ids.tolist() == [5, 5, 5, 0]
    assert ctx.cu_q.tolist() == [0, 1, 2, 3, 4] and ctx.seq_lens.tolist() == [4, 4, 4, 0]
    assert ctx.logit_rows.tolist() == [0, 1, 2, 0]
    assert ctx.temperatures.tolist()[:4] == pytest.approx([0.7, 0.7, 0.7, 0.0])
    views = [ctx.token_ids, ctx.positions, ctx.req_index, ctx.logit_rows, ctx.cu_q, ctx.seq_lens, ctx.state_slots,
             ctx.first_portion, *ctx.group_slot_mapping, ctx.temperatures, ctx.uniforms]
    spans = sorted((v.data_ptr(), v.data_ptr() + v.numel() * 4) for v in views)
    assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:])), "staging regions overlap"
    for e in entries:
        cache.release_allocation(e.request_id)
    # and the same through the engine: four requests decoding under a budget of three tokens a step
    cfg, w = P.read_model(models["B"])
    eng2 = engine(models["B"], "B", max_num_batched_tokens=3, max_num_seqs=4)
    prompts = [tiny.random_tokens(320, n, 70 + n) for n in (4, 2, 5, 3)]
    outs = eng2.generate(prompts, SamplingParams(max_tokens=6))
    for p, o in zip(prompts, outs):
        assert o == P.greedy(cfg, w, p, 6)
    eng2.runner.cache.check()


def test_more_sampled_rows_than_requests_are_refused_before_pages_are_taken(models):
    eng = engine(models["A"], "A", max_num_seqs=2)
    run, cache = eng.runner, eng.runner.cache
    cache.add_request("a")
    free = cache.free_pages()
    with pytest.raises(BatchError, match="rows to sample"):
        run.step_and_sample([StepEntry("a", [1, 2, 3, 4], [0, 1, 2])], [0.0] * 3, [0.0] * 3)
    assert cache.free_pages() == free
    assert run.step([StepEntry("a", [1, 2, 3, 4], [0, 1, 2])]).shape[0] == 3      # logits alone may be wanted anywhere


def test_a_step_that_raises_gives_its_pages_back(models, monkeypatch):
    eng = engine(models["A"], "A")
    run, cache = eng.runner, eng.runner.cache
    cache.add_request("a")
    run.step([StepEntry("a", [1, 2, 3])])
    free = cache.free_pages()
    monkeypatch.setattr(run.model, "forward", lambda ctx: (_ for _ in ()).throw(RuntimeError("kernel refused")))
    with pytest.raises(RuntimeError, match="kernel refused"):
        run.step([StepEntry("a", list(range(40)), [39])])
    assert cache.free_pages() == free and cache.num_computed("a") == 3
    cache.check()


def test_a_fault_recorded_on_the_device_fails_the_requests_that_ran(models):
    """The kernels' error word is read every 32 steps and before a request is reported finished.  When it
    is set, every request that ran since it was last read clean fails, with its pages and slot given
    back, and the engine goes on with new requests.  The fault is injected on the host: the stand-in
    kernel set raises from ``check_device_errors`` as the CUDA kernel set does for a non-zero word."""
    class Faulty(ReferenceKernels):
        armed = False

        def check_device_errors(self):
            if self.armed:
                self.armed = False
                raise KernelError("a kernel gave up waiting on a barrier (code 7); its output is not valid")

    kernels = Faulty()
    opts = EngineOptions(dtype="float32", device="cpu", page_size=16, num_pages=40, max_num_seqs=4, max_num_batched_tokens=64)
    eng = Engine.from_model_dir(models["A"], opts, kernels=kernels)
    eng.add_request(Request("long", [1, 2, 3], SamplingParams(max_tokens=60)))
    eng.add_request(Request("short", [4, 5], SamplingParams(max_tokens=3)))
    eng.step()
    kernels.armed = True
    failed = []
    for _ in range(10):
        res = eng.step()
        failed += list(res.failed_requests)
        assert "short" not in res.completed_requests          # it is not reported finished on poisoned output
        if eng.is_done():
            break
    assert sorted(failed) == ["long", "short"]
    for rid in ("long", "short"):
        r = eng.scheduler.get_request(rid)
        assert r.state is RequestState.FAILED and "code 7" in r.error
    assert eng.is_done() and eng.runner.cache.free_pages() == [40]
    eng.runner.cache.check()
    assert len(eng.generate([[7, 8, 9]], SamplingParams(max_tokens=4))[0]) == 4
