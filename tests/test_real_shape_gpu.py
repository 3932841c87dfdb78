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
    write_random_model(cfg, 3, path)
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
