"""Weights: the safetensors reader, the loader's one error, dtypes, and the random writer."""
import json
import os
import struct

import pytest
import torch

from infurnace_b200.errors import WeightError
from infurnace_b200.models import config_from_dict, plan_for
from infurnace_b200.weights.loader import load_weights
from infurnace_b200.weights.random_init import write_random_model
from infurnace_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
import tiny


@pytest.fixture()
def folder(tmp_path):
    cfg = config_from_dict(tiny.TINY["B"]["config"])
    return cfg, write_random_model(cfg, 5, str(tmp_path / "m"))


def _rewrite(folder, edit):
    from safetensors.torch import load_file, save_file
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    edit(t)
    save_file(t, path)


def test_reader_agrees_with_the_library(folder):
    from safetensors.torch import load_file
    cfg, d = folder
    theirs = load_file(os.path.join(d, "model.safetensors"))
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    assert set(f.entries) == set(theirs)
    for k, v in theirs.items():
        assert torch.equal(f.tensor(k), v)
    f.close()


def test_random_weights_are_a_function_of_seed_and_name(tmp_path):
    cfg = config_from_dict(tiny.TINY["A"]["config"])
    a = load_weights(write_random_model(cfg, 1, str(tmp_path / "a"), "float32"), plan_for(cfg), torch.float32, "cpu")
    b = load_weights(write_random_model(cfg, 1, str(tmp_path / "b"), "float32"), plan_for(cfg), torch.float32, "cpu")
    c = load_weights(write_random_model(cfg, 2, str(tmp_path / "c"), "float32"), plan_for(cfg), torch.float32, "cpu")
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    w = a["model.layers.0.mlp.up_proj.weight"]
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    n = a["model.layers.1.input_layernorm.weight"]
    assert abs(float(n.mean()) - 1.0) < 0.05 and 0.05 < float(n.std()) < 0.15
    # a layer's tensor does not change when the model gets more layers
    cfg3 = config_from_dict({**tiny.TINY["A"]["config"], "num_hidden_layers": 3})
    d3 = load_weights(write_random_model(cfg3, 1, str(tmp_path / "d"), "float32"), plan_for(cfg3), torch.float32, "cpu")
    assert torch.equal(d3["model.layers.1.mlp.up_proj.weight"], a["model.layers.1.mlp.up_proj.weight"])


def test_one_error_lists_missing_unexpected_and_wrong_shapes(folder):
    cfg, d = folder

    def edit(t):
        del t["model.layers.1.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.9.extra.weight"] = torch.zeros(2)
        t["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(cfg.head_dim + 1, dtype=torch.bfloat16)
        t["model.embed_tokens.weight"] = torch.zeros((cfg.vocab_size, cfg.hidden_size), dtype=torch.int32)

    _rewrite(d, edit)
    with pytest.raises(WeightError) as e:
        load_weights(d, plan_for(cfg), torch.bfloat16, "cpu")
    msg = str(e.value)
    assert "missing tensors (2): model.layers.1.mlp.up_proj.weight, model.norm.weight" in msg
    assert "unexpected tensors (1): model.layers.9.extra.weight" in msg
    assert f"model.layers.0.self_attn.q_norm.weight: expected ({cfg.head_dim},), got ({cfg.head_dim + 1},)" in msg
    assert "model.embed_tokens.weight: expected a floating dtype, got I32" in msg


def test_nothing_is_read_before_the_check(folder, monkeypatch):
    cfg, d = folder
    _rewrite(d, lambda t: t.pop("model.norm.weight"))
    reads = []
    monkeypatch.setattr(SafetensorsFile, "tensor", lambda self, name: reads.append(name))
    with pytest.raises(WeightError):
        load_weights(d, plan_for(cfg), torch.bfloat16, "cpu")
    assert reads == []       # the reference checks before any cast too (tests/test_model_weights.py:80-103)


def test_tied_model_takes_a_stored_head_only_as_a_copy_of_the_embedding(tmp_path):
    """The reference demands that head and embedding be one object (weights.py:68, model.py:34-36): a folder
    of a tied model that also stores lm_head.weight loads if the two are equal bit for bit, and the head
    then reads the embedding table; a head that differs, in value, dtype or shape, is an error."""
    cfg = config_from_dict(tiny.TINY["A"]["config"])
    plan = plan_for(cfg)
    d = write_random_model(cfg, 1, str(tmp_path / "a"))
    _rewrite(d, lambda t: t.__setitem__("lm_head.weight", t["model.embed_tokens.weight"].clone()))
    w = load_weights(d, plan, torch.bfloat16, "cpu")
    assert "lm_head.weight" not in w and plan.lm_head.weight == "model.embed_tokens.weight"

    def nudge(t):
        h = t["model.embed_tokens.weight"].clone()
        h[3, 5] += 1.0
        t["lm_head.weight"] = h
    _rewrite(d, nudge)
    with pytest.raises(WeightError, match="unexpected tensors.*lm_head.weight.*differ"):
        load_weights(d, plan, torch.bfloat16, "cpu")
    _rewrite(d, lambda t: t.__setitem__("lm_head.weight", t["model.embed_tokens.weight"].float()))
    with pytest.raises(WeightError, match="lm_head.weight: stored beside"):
        load_weights(d, plan, torch.bfloat16, "cpu")
    # an untied model still needs its head, and a tied one accepts no other stranger
    _rewrite(d, lambda t: (t.pop("lm_head.weight"), t.__setitem__("extra.weight", torch.zeros(2))))
    with pytest.raises(WeightError, match="unexpected tensors.*extra.weight"):
        load_weights(d, plan, torch.bfloat16, "cpu")


def test_dtype_policy(tmp_path):
    cfg = config_from_dict(tiny.TINY["C"]["config"])
    d = write_random_model(cfg, 1, str(tmp_path / "c"), store_dtype="bfloat16", norm_dtype="float32")
    w = load_weights(d, plan_for(cfg), torch.bfloat16, "cpu")
    assert w["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16        # bfloat16 stays
    assert w["model.norm.weight"].dtype == torch.float32                          # stored in 32-bit stays so
    w32 = load_weights(d, plan_for(cfg), torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in w32.values())
    assert torch.equal(w32["model.layers.0.mlp.up_proj.weight"], w["model.layers.0.mlp.up_proj.weight"].float())
    _rewrite(d, lambda t: t.__setitem__("model.norm.weight", t["model.norm.weight"].half()))
    assert load_weights(d, plan_for(cfg), torch.bfloat16, "cpu")["model.norm.weight"].dtype == torch.bfloat16


def test_integer_tables_become_int32(tmp_path):
    path = str(tmp_path / "t.safetensors")
    write_safetensors(path, [("table", torch.arange(6, dtype=torch.int64).view(2, 3))])
    from infurnace_b200.config.specs import TensorSpec
    from infurnace_b200.weights.loader import target_dtype, check_inventory
    f = SafetensorsFile(path)
    check_inventory(f.entries, {"table": TensorSpec((2, 3), "int")})
    assert target_dtype("I64", "int", torch.bfloat16) == torch.int32
    assert f.tensor("table").tolist() == [[0, 1, 2], [3, 4, 5]]
    f.close()


def test_sharded_folder_with_index(folder, tmp_path):
    from safetensors.torch import load_file, save_file
    cfg, d = folder
    t = load_file(os.path.join(d, "model.safetensors"))
    names = sorted(t)
    half = len(names) // 2
    os.remove(os.path.join(d, "model.safetensors"))
    save_file({k: t[k] for k in names[:half]}, os.path.join(d, "model-00001-of-00002.safetensors"))
    save_file({k: t[k] for k in names[half:]}, os.path.join(d, "model-00002-of-00002.safetensors"))
    index = {"weight_map": {k: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                            for i, k in enumerate(names)}}
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump(index, f)
    w = load_weights(d, plan_for(cfg), torch.bfloat16, "cpu")
    assert all(torch.equal(w[k], t[k]) for k in names)


def test_broken_files(tmp_path):
    p = tmp_path / "x.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(WeightError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(WeightError, match="header length"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(WeightError, match="data offsets"):
        SafetensorsFile(str(p))
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(WeightError, match="no .safetensors"):
        load_weights(str(empty), None, torch.float32, "cpu")


def test_random_values_are_counter_based_and_roughly_normal():
    from infurnace_b200.weights.random_init import normal_values, tensor_seed
    s = tensor_seed(3, "model.layers.0.mlp.up_proj.weight")
    a = normal_values(s, 200_000, 0.0, 0.02)
    assert torch.equal(a[:1000], normal_values(s, 1000, 0.0, 0.02))          # element i does not depend on n
    assert abs(float(a.mean())) < 2e-4 and abs(float(a.std()) - 0.02) < 2e-4
    assert 0.66 < float((a.abs() < 0.02).float().mean()) < 0.70              # one sigma holds about 68 %
    assert not torch.equal(a[:1000], normal_values(tensor_seed(3, "model.layers.1.mlp.up_proj.weight"), 1000, 0.0, 0.02))
    b = normal_values(s, 1000, 1.0, 0.1)
    assert abs(float(b.mean()) - 1.0) < 0.02


def test_random_weights_without_a_folder_equal_the_folders(tmp_path):
    """``Engine.from_random`` without a work folder draws the tensors where the engine runs (here through
    the stand-in kernel set) and gives the engine the same tensors as writing the folder and loading it."""
    from kernel_refs import ReferenceKernels
    from infurnace_b200.engine import Engine, EngineOptions, SamplingParams
    cfg = config_from_dict(tiny.TINY["B"]["config"])
    opts = dict(dtype="float32", device="cpu", page_size=8, num_pages=32, max_num_seqs=2, max_num_batched_tokens=64)
    a = Engine.from_random(cfg, 4, EngineOptions(**opts), kernels=ReferenceKernels())
    b = Engine.from_random(cfg, 4, EngineOptions(**opts), kernels=ReferenceKernels(), workdir=str(tmp_path / "m"))
    prompt = tiny.random_tokens(320, 12, 1)
    assert a.generate([prompt], SamplingParams(max_tokens=8)) == b.generate([prompt], SamplingParams(max_tokens=8))
    la, lb = a.runner.model.layers[1], b.runner.model.layers[1]
    assert torch.equal(la.mixer.w_qkv, lb.mixer.w_qkv) and torch.equal(la.ffn.w_down, lb.ffn.w_down)
    assert torch.equal(a.runner.model.lm_head.weight, b.runner.model.lm_head.weight)
