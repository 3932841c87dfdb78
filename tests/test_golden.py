"""The plain implementation (and the engine) against the reference's own model code.

tests/golden/reference_logits.npz holds the logits that src/infurnace/executor/tinygrad/model.py of
tylerguest/infurnace, imported unmodified, gives on two tiny models; tests/golden/make_golden.py wrote
it, with tinygrad's Tensor replaced by the torch stand-in of tests/golden/tinygrad_standin.py.  So the
structure of the computation is the reference's, the elementary operations are torch's.  With
INFURNACE_REFERENCE_SRC set to the src folder of a checkout, the file is also recomputed and compared."""
import json
import os
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as P

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
sys.path.insert(0, GOLDEN)
import golden_model as G          # noqa: E402


@pytest.fixture(scope="module")
def stored():
    return np.load(os.path.join(GOLDEN, "reference_logits.npz"))


def _config_json(cfg):
    d = {k: v for k, v in cfg.items() if k not in ("seed", "tokens")}
    d["architectures"] = ["Qwen3ForCausalLM"]
    return d


@pytest.mark.parametrize("name", list(G.MODELS))
def test_plain_implementation_equals_the_references_model(stored, name):
    cfg = G.MODELS[name]
    logits = P.forward(_config_json(cfg), G.weights(cfg), G.tokens(cfg))
    whole = torch.from_numpy(stored[f"{name}/whole"])
    assert logits.shape == whole.shape
    err = float((logits - whole).abs().max())
    print(f"\n{name}: plain against the reference's whole-sequence forward: {err:.2e} (largest logit {float(whole.abs().max()):.2f})")
    assert err <= 5e-6
    # through the reference's cache (a portion, a portion on top of it, then single tokens): the same places,
    # up to the float16 rounding of the keys and values it stores (buffers.py:22)
    cached, places = torch.from_numpy(stored[f"{name}/cached"]), stored[f"{name}/cached_places"]
    assert float((logits[places] - cached).abs().max()) <= 6e-3
    # far below what a wrong position, mask or pairing does: shifting the rows by one place
    assert float((logits[places - 1] - cached).abs().max()) > 0.2


def test_stored_outputs_are_what_the_reference_gives_now(stored):
    src = os.environ.get("INFURNACE_REFERENCE_SRC")
    if not src or not os.path.isdir(os.path.join(src, "infurnace")):
        pytest.skip("set INFURNACE_REFERENCE_SRC to the src folder of a tylerguest/infurnace checkout")
    import make_golden
    for name, cfg in G.MODELS.items():
        whole, cached, places = make_golden.run(cfg, os.path.abspath(src))
        assert np.abs(whole - stored[f"{name}/whole"]).max() <= 1e-6
        assert np.abs(cached - stored[f"{name}/cached"]).max() <= 1e-6
        assert (places == stored[f"{name}/cached_places"]).all()


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(G.MODELS))
def test_engine_equals_the_references_model(stored, name, tmp_path):
    """The engine itself, in float32, whole and token by token, against the reference's logits."""
    from safetensors.torch import save_file
    import tiny
    from infurnace_b200.engine.loading import EngineOptions, build_runner
    cfg = G.MODELS[name]
    d = str(tmp_path / name)
    os.makedirs(d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(_config_json(cfg), f)
    save_file({k: v.contiguous() for k, v in G.weights(cfg).items()}, os.path.join(d, "model.safetensors"))
    toks = G.tokens(cfg)
    whole = torch.from_numpy(stored[f"{name}/whole"])
    runner = build_runner(d, EngineOptions(dtype="float32", page_size=16, num_pages=8, max_num_seqs=2,
                                           max_num_batched_tokens=64))[2]
    reqs = {"a": toks}
    for steps in (tiny.schedule_whole(reqs), tiny.schedule_bulk_tail(reqs, tail=len(toks) - 1)):
        out = tiny.collect(steps, tiny.run_inprocess(runner, steps), cfg["vocab_size"])["a"]
        assert float((out - whole).abs().max()) <= 2e-5
