"""The kernels at the sizes of the real checkpoints: the layer sizes of Qwen3-0.6B (heads of 128,
hidden 1024, 16 query and 8 key/value heads, intermediate 3072, vocabulary 151,936, tied head) with two
layers and random weights, against the plain implementation: a prompt in one step, the same in
portions with a decoded tail, in float32 and in bfloat16.  This is where the tcgen05 product, the
TMA-fed attention and the decode product run at the sizes the benchmark times."""
import json
import os

import pytest
import torch

import plain_qwen3 as P
import tiny

pytestmark = pytest.mark.gpu


# the layer sizes of the three checkpoints the benchmarks name; the two large ones with one layer and a small
# vocabulary, so that the plain implementation on the CPU stays within seconds
SHAPES = {
    "0.6b": ("qwen3-0.6b.json", dict(num_hidden_layers=2)),
    "8b": ("qwen3-8b.json", dict(num_hidden_layers=1, vocab_size=4096)),          # 32 / 8 heads, hidden 4096, mlp 12288
    "32b": ("qwen3-32b.json", dict(num_hidden_layers=1, vocab_size=4096)),        # 64 / 8 heads, hidden 5120, mlp 25600
}


@pytest.fixture(scope="module", params=list(SHAPES))
def model(request, tmp_path_factory):
    from infurnace_b200.models import config_from_dict
    from infurnace_b200.weights.random_init import write_random_model
    from safetensors.torch import load_file, save_file
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    file_name, changes = SHAPES[request.param]
    with open(os.path.join(root, "configs", file_name)) as f:
        d = json.load(f)
    d.update(changes)
    cfg = config_from_dict(d)
    path = str(tmp_path_factory.mktemp("real") / "m")
    from infurnace_b200.kernels import load_cuda_kernels
    write_random_model(cfg, 3, path, kernels=load_cuda_kernels())        # drawn on the device: the same values, in seconds
    file = os.path.join(path, "model.safetensors")
    t = load_file(file)
    for k in list(t):                      # peaked attention, as in the tiny models
        if k.endswith("q_norm.weight"):
            t[k] = (t[k].float() * 3.0).to(t[k].dtype)
    save_file(t, file)
    cfgd, w = P.read_model(path)
    toks = tiny.random_tokens(cfgd["vocab_size"], 330, 77)
    return path, cfgd, toks, P.forward(cfgd, w, toks)


@pytest.mark.parametrize("dtype,tolerance", [("float32", 2e-5), ("bfloat16", 0.05)])   # times the size of the largest logit
def test_real_layer_sizes(model, dtype, tolerance):
    from infurnace_b200.engine.loading import EngineOptions, build_runner
    path, cfg, toks, ref = model
    opts = EngineOptions(dtype=dtype, page_size=16, num_pages=64, max_num_seqs=2, max_num_batched_tokens=512)
    runner = build_runner(path, opts)[2]
    reqs = {"a": toks}
    whole = tiny.schedule_whole(reqs)
    cut = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:200], "want": list(range(200))}], "end": []},
           {"step": 1, "entries": [{"id": "a", "tokens": toks[200:297], "want": list(range(97))}], "end": []},
           {"step": 2, "entries": [{"id": "a", "tokens": toks[297:299], "want": [0, 1]}], "end": []}]
    cut += [{"step": 3 + i, "entries": [{"id": "a", "tokens": [toks[299 + i]], "want": [0]}],
             "end": ["a"] if 299 + i == len(toks) - 1 else []} for i in range(len(toks) - 299)]
    scale = float(ref.abs().max())
    for steps in (whole, cut):
        out = tiny.collect(steps, tiny.run_inprocess(runner, steps), cfg["vocab_size"])["a"]
        err = (out - ref).abs().max(dim=-1).values
        assert float(err.max()) <= tolerance * max(1.0, scale), (int(err.argmax()), float(err.max()), scale)
    runner.rt.kernels.check_device_errors()


# ----------------------------------------------------------------------------------------------------------------
# Every way of cutting the work where the product's own kernels meet: head size 128 and pages of 16, so that prompt
# portions run on the tcgen05 attention kernel beside decoded tokens on the TMA-fed small-q kernel in one step,
# products of more than 64 rows on tcgen05 beside few-row ones (and, from 17 rows, o and down on tcgen05 with their k
# range shared by a cluster), norms folded into the products of steps up to 128 rows and run as kernels above.  The layer sizes are Qwen3-0.6B's, with two layers and a vocabulary of 4,096.
# ----------------------------------------------------------------------------------------------------------------
CUT_LENS = [137, 300, 64, 19, 285, 150, 1, 2, 328]


@pytest.fixture(scope="module")
def small_06b(tmp_path_factory):
    from infurnace_b200.models import config_from_dict
    from infurnace_b200.weights.random_init import write_random_model
    from safetensors.torch import load_file, save_file
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(root, "configs", "qwen3-0.6b.json")) as f:
        d = json.load(f)
    d.update(num_hidden_layers=2, vocab_size=4096)
    path = str(tmp_path_factory.mktemp("cut") / "m")
    from infurnace_b200.kernels import load_cuda_kernels
    write_random_model(config_from_dict(d), 5, path, kernels=load_cuda_kernels())
    file = os.path.join(path, "model.safetensors")
    t = load_file(file)
    for k in list(t):
        if k.endswith("q_norm.weight"):
            t[k] = (t[k].float() * 3.0).to(t[k].dtype)
    save_file(t, file)
    cfg, w = P.read_model(path)
    reqs = {f"r{i}": tiny.random_tokens(cfg["vocab_size"], n, 300 + i) for i, n in enumerate(CUT_LENS)}
    ref = {r: P.forward(cfg, w, t) for r, t in reqs.items()}
    return path, cfg, w, reqs, ref


@pytest.mark.parametrize("dtype,tolerance", [("float32", 2e-5), ("bfloat16", 0.04)])   # times the size of the largest logit
@pytest.mark.parametrize("mode", ["whole", "bulk_tail", "portions", "mixed"])
def test_cutting_modes_at_the_real_head_size(small_06b, mode, dtype, tolerance):
    from infurnace_b200.engine.loading import EngineOptions, build_runner
    path, cfg, w, reqs, ref = small_06b
    steps = {"whole": tiny.schedule_whole, "bulk_tail": lambda r: tiny.schedule_bulk_tail(r, tail=32),
             "portions": lambda r: tiny.schedule_portions(r, seed=3),
             "mixed": lambda r: tiny.schedule_mixed(r, max_live=4, max_tokens=1024, seed=4, tail=20,
                                                    sizes=(2, 5, 13, 40, 70, 130))}[mode](reqs)
    opts = EngineOptions(dtype=dtype, page_size=16, num_pages=1024 // 16, max_num_seqs=4, max_num_batched_tokens=1024)
    runner = build_runner(path, opts)[2]
    K = runner.rt.kernels
    before = (K.tc_attention_calls, K.small_q_tma_calls, K.fused_qkv_calls, K.tc_shared_k_calls, K.tc_folded_calls)
    out = tiny.collect(steps, tiny.run_inprocess(runner, steps), cfg["vocab_size"])
    runner.cache.check()
    assert runner.cache.free_pages() == [64]
    if mode == "mixed":          # four live requests of up to 384 tokens (rounded) in 1,024: pages were used again
        assert sum(-(-n // 16) for n in CUT_LENS) > 64
    scale = max(float(r.abs().max()) for r in ref.values())
    worst = ("", 0, 0.0)
    for rid in reqs:
        err = (out[rid] - ref[rid]).abs().max(dim=-1).values
        pos = int(err.argmax())
        if float(err[pos]) > worst[2]:
            worst = (rid, pos, float(err[pos]))
    print(f"\n0.6B widths, {mode}, {dtype}: largest error {worst[2]:.3e} (request {worst[0]}, position {worst[1]}); "
          f"largest logit {scale:.3f}; bound {tolerance * max(1.0, scale):.3e}")
    assert worst[2] <= tolerance * max(1.0, scale), f"{mode} {dtype}: first look at request {worst[0]} position {worst[1]}: {worst[2]}"
    if dtype == "bfloat16":
        assert K.tc_attention_calls > before[0], "the tcgen05 attention kernel did not run"
        if mode != "whole":
            assert K.small_q_tma_calls > before[1], "the TMA-fed small-q kernel did not run"
            assert K.fused_qkv_calls > before[2], "the q | k | v product with norm, rotation and store in its epilogue did not run"
        if mode in ("portions", "mixed"):          # steps of some tens of tokens
            assert K.tc_shared_k_calls > before[3], "no tcgen05 product shared its k range in a cluster"
            assert K.tc_folded_calls > before[4], "no tcgen05 product took or made a folded norm"
    K.check_device_errors()


_LONG = {}


@pytest.mark.parametrize("dtype,tolerance", [("float32", 2e-5), ("bfloat16", 0.05)])
def test_a_long_context_in_the_benchmarks_regime(small_06b, dtype, tolerance):
    """One request prefilled to 4,000 tokens in portions of 2,048 and 1,952, then 64 tokens decoded one by one beside
    three shorter requests that prefill and decode meanwhile; logits wanted at a few dozen places only.  This is the
    regime the benchmark times: thousands of keys per request, the context split over CTAs, the 2,048-token step on
    the wide tcgen05 tile shapes, a second portion on top of the first."""
    from infurnace_b200.engine.loading import EngineOptions, build_runner
    path, cfg, w, _, _ = small_06b
    vocab = cfg["vocab_size"]
    long = tiny.random_tokens(vocab, 4064, 900)
    short = {f"s{i}": tiny.random_tokens(vocab, n, 910 + i) for i, n in enumerate((96, 150, 40))}
    if "ref" not in _LONG:          # the plain implementation's 4,064 tokens take a quarter of a minute: once for both dtypes
        _LONG["ref"] = {"L": P.forward(cfg, w, long), **{r: P.forward(cfg, w, t) for r, t in short.items()}}
    ref = _LONG["ref"]
    steps = [{"step": 0, "entries": [{"id": "L", "tokens": long[:2048], "want": [0, 1000, 2047]}], "end": []},
             {"step": 1, "entries": [{"id": "L", "tokens": long[2048:4000], "want": [0, 1951]},
                                     {"id": "s0", "tokens": short["s0"][:90], "want": [89]}], "end": []}]
    done = {"s0": 90, "s1": 0, "s2": 0}
    for i in range(64):
        entries = [{"id": "L", "tokens": [long[4000 + i]], "want": [0]}]
        for rid, toks in short.items():
            s = done[rid]
            if s >= len(toks) or (rid == "s2" and i < 10):        # s2 joins later
                continue
            n = 1 if len(toks) - s <= 20 else min(len(toks) - s - 20, (70, 33, 9)[i % 3])
            entries.append({"id": rid, "tokens": toks[s:s + n], "want": [n - 1]})
            done[rid] = s + n
        ended = [rid for rid in short if done[rid] == len(short[rid]) and any(e["id"] == rid for e in entries)]
        if i == 63:
            ended.append("L")
        steps.append({"step": 2 + i, "entries": entries, "end": ended})
    assert all(done[r] == len(t) for r, t in short.items())
    opts = EngineOptions(dtype=dtype, page_size=16, num_pages=(4064 + 96 + 160 + 48) // 16 + 2, max_num_seqs=4,
                         max_num_batched_tokens=2048)
    runner = build_runner(path, opts)[2]
    K = runner.rt.kernels
    outputs = tiny.run_inprocess(runner, steps)
    runner.cache.check()
    scale = float(ref["L"].abs().max())
    worst = ("", 0, 0.0)
    position = {"L": 0, "s0": 0, "s1": 0, "s2": 0}
    rows_checked = 0
    for st in steps:
        out = outputs.get(st["step"])
        row = 0
        for e in st["entries"]:
            for wnt in e["want"]:
                pos = position[e["id"]] + wnt
                err = float((out[row] - ref[e["id"]][pos]).abs().max())
                if err > worst[2]:
                    worst = (e["id"], pos, err)
                row += 1
                rows_checked += 1
            position[e["id"]] += len(e["tokens"])
    print(f"\nlong context, {dtype}: {rows_checked} rows, largest error {worst[2]:.3e} (request {worst[0]}, position "
          f"{worst[1]}); largest logit {scale:.3f}; bound {tolerance * max(1.0, scale):.3e}")
    assert worst[2] <= tolerance * max(1.0, scale), worst
    if dtype == "bfloat16":
        assert K.tc_attention_calls > 0 and K.small_q_tma_calls > 0
    K.check_device_errors()
