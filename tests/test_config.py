"""Configuration and registry (no GPU, no torch needed by the code under test)."""
import json
import subprocess
import sys

import pytest

from infurnace_b200.config import Qwen3Config
from infurnace_b200.errors import ModelConfigError
from infurnace_b200.models import config_from_dict, known_architectures, plan_for, read_config, register_architecture
import tiny

BASE = tiny.TINY["A"]["config"]


def test_reads_every_size_from_the_file():
    for name, spec in tiny.TINY.items():
        d = spec["config"]
        cfg = config_from_dict(d)
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                    "num_key_value_heads", "head_dim", "rope_theta", "rms_norm_eps", "max_position_embeddings"):
            assert getattr(cfg, key) == d[key], (name, key)
        assert cfg.tie_word_embeddings == d["tie_word_embeddings"]
        assert cfg.q_size == d["num_attention_heads"] * d["head_dim"]
        assert cfg.gqa_ratio == d["num_attention_heads"] // d["num_key_value_heads"]


def test_defaults_of_absent_keys():
    d = {k: v for k, v in BASE.items() if k not in ("num_key_value_heads", "head_dim", "rope_theta", "rms_norm_eps",
                                                    "tie_word_embeddings")}
    cfg = config_from_dict(d)
    assert cfg.num_key_value_heads == cfg.num_attention_heads
    assert cfg.head_dim == cfg.hidden_size // cfg.num_attention_heads
    assert cfg.rope_theta == 10000.0 and cfg.rms_norm_eps == 1e-6 and cfg.tie_word_embeddings is False


def test_config_is_immutable():
    cfg = config_from_dict(BASE)
    with pytest.raises(Exception):
        cfg.hidden_size = 1


def test_round_trip_through_to_dict():
    for spec in tiny.TINY.values():
        cfg = config_from_dict(spec["config"])
        assert config_from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg


@pytest.mark.parametrize("change,fragment", [
    ({"num_key_value_heads": 3}, "divisible"),
    ({"head_dim": 15}, "even"),
    ({"rope_theta": 0.0}, "rope_theta"),
    ({"rms_norm_eps": float("nan")}, "rms_norm_eps"),
    ({"attention_bias": True}, "attention_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"hidden_size": None}, "hidden_size"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"layer_types": ["full_attention", "sliding_attention"]}, "sliding_window"),
    ({"layer_types": ["full_attention", "banded"]}, "unknown layer type"),
])
def test_bad_values_are_refused(change, fragment):
    with pytest.raises(ModelConfigError, match=fragment):
        config_from_dict({**BASE, **change})


def test_window_keys():
    cfg = config_from_dict({**BASE, "use_sliding_window": True, "sliding_window": 8, "max_window_layers": 1})
    assert cfg.layer_types == ("full_attention", "sliding_attention") and cfg.sliding_window == 8
    cfg = config_from_dict({**BASE, "use_sliding_window": False, "sliding_window": 8})
    assert cfg.sliding_window is None and set(cfg.layer_types) == {"full_attention"}
    plan = plan_for(config_from_dict(tiny.TINY["B"]["config"]))
    assert [l.mixer.window for l in plan.layers] == [None, 24, None]


def test_registry():
    assert "Qwen3ForCausalLM" in known_architectures()
    with pytest.raises(ModelConfigError, match="unknown architecture 'Nope'.*Qwen3ForCausalLM"):
        config_from_dict({**BASE, "architectures": ["Nope"]})
    with pytest.raises(ModelConfigError, match="architectures"):
        config_from_dict({k: v for k, v in BASE.items() if k != "architectures"})
    with pytest.raises(ModelConfigError, match="already registered"):
        register_architecture("Qwen3ForCausalLM", Qwen3Config, lambda c: None)


def test_plan_names_every_tensor():
    for name, spec in tiny.TINY.items():
        cfg = config_from_dict(spec["config"])
        t = plan_for(cfg).tensors()
        # 2 + 11 per layer, + 1 for an untied head (the reference's inventory, src/infurnace/models/qwen3.py:37-60)
        assert len(t) == 2 + 11 * cfg.num_hidden_layers + (0 if cfg.tie_word_embeddings else 1)
        assert t["model.layers.0.self_attn.q_proj.weight"].shape == (cfg.q_size, cfg.hidden_size)
        assert t["model.layers.0.self_attn.k_norm.weight"].shape == (cfg.head_dim,)
        assert t["model.layers.0.mlp.down_proj.weight"].shape == (cfg.hidden_size, cfg.intermediate_size)
        assert ("lm_head.weight" in t) == (not cfg.tie_word_embeddings)


def test_schedule_is_data():
    from infurnace_b200.config.specs import LayerCall
    import dataclasses
    plan = plan_for(config_from_dict(tiny.TINY["A"]["config"]))
    assert [c.layer for c in plan.resolved_schedule()] == [0, 1] and [c.cache for c in plan.resolved_schedule()] == [0, 1]
    twice = dataclasses.replace(plan, schedule=(LayerCall(0), LayerCall(1, cache=1), LayerCall(0), LayerCall(1, cache=1, store=False)))
    r = twice.resolved_schedule()
    assert [c.cache for c in r] == [0, 1, 2, 1] and [c.store for c in r] == [True, True, True, False]
    with pytest.raises(ValueError):
        dataclasses.replace(plan, schedule=(LayerCall(0, cache=5, store=False),)).resolved_schedule()
    with pytest.raises(ValueError):
        dataclasses.replace(plan, schedule=(LayerCall(7),)).resolved_schedule()


def test_read_config_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(tiny.TINY["B"]["config"]))
    assert read_config(str(tmp_path)).hidden_size == 96
    with pytest.raises(ModelConfigError):
        read_config(str(tmp_path / "missing"))


def test_model_contract_imports_without_torch():
    code = ("import sys; import infurnace_b200.models, infurnace_b200.config, infurnace_b200.cache; "
            "assert 'torch' not in sys.modules, 'torch was imported'")
    root = str(__import__("pathlib").Path(__file__).resolve().parents[1])
    subprocess.run([sys.executable, "-c", code], check=True, cwd=root)
