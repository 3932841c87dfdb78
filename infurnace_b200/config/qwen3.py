"""Typed configuration of the Qwen3 dense decoder, read from config.json's own keys.

The reference derives the same quantities from GGUF metadata and pins each of them to
the 0.6B checkpoint (src/infurnace/models/qwen3.py:12-35,62-96); here every value is
read from the file and any consistent combination is accepted.  The consistency rules
are the reference's: query heads divisible by key/value heads (qwen3.py:76), an even
head size for the rotation (qwen3.py:78), finite positive rope base and epsilon
(qwen3.py:79-80).  Options that the architecture's code path does not have (attention
bias, another activation, scaled rotary frequencies) are refused with an error, never
ignored (qwen3.py:94-95 fixes them).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, asdict
from typing import Any, Mapping, Optional, Tuple

from ..errors import ModelConfigError

FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


def _need(d: Mapping[str, Any], key: str, typ) -> Any:
    if key not in d or d[key] is None:
        raise ModelConfigError(f"config.json lacks required key {key!r}")
    v = d[key]
    if typ is int and (isinstance(v, bool) or not isinstance(v, int)):
        raise ModelConfigError(f"config.json key {key!r} must be an integer, got {v!r}")
    if typ is float and (isinstance(v, bool) or not isinstance(v, (int, float))):
        raise ModelConfigError(f"config.json key {key!r} must be a number, got {v!r}")
    return typ(v)


@dataclass(frozen=True)
class Qwen3Config:
    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rope_theta: float
    rms_norm_eps: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    hidden_act: str
    attention_bias: bool
    sliding_window: Optional[int]
    layer_types: Tuple[str, ...]

    # ---- derived sizes
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def gqa_ratio(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    # ---- construction
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen3Config":
        if not isinstance(d, Mapping):
            raise ModelConfigError("config.json must hold a JSON object")
        archs = d.get("architectures")
        if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
            raise ModelConfigError("config.json lacks required key 'architectures'")
        hidden = _need(d, "hidden_size", int)
        heads = _need(d, "num_attention_heads", int)
        layers = _need(d, "num_hidden_layers", int)
        kv_heads = d.get("num_key_value_heads")
        kv_heads = heads if kv_heads is None else _need(d, "num_key_value_heads", int)
        if heads < 1 or kv_heads < 1 or layers < 1 or hidden < 1:
            raise ModelConfigError("sizes in config.json must be positive")
        if d.get("head_dim") is None:
            if hidden % heads:
                raise ModelConfigError("head_dim is absent and hidden_size is not divisible by num_attention_heads")
            head_dim = hidden // heads
        else:
            head_dim = _need(d, "head_dim", int)
        # rope base: flat key, or the nested form that newer files use
        rope_params = d.get("rope_parameters") or {}
        if d.get("rope_theta") is not None:
            theta = _need(d, "rope_theta", float)
        elif isinstance(rope_params, Mapping) and rope_params.get("rope_theta") is not None:
            theta = float(rope_params["rope_theta"])
        else:
            theta = 10000.0
        scaling = d.get("rope_scaling")
        if scaling is None and isinstance(rope_params, Mapping):
            rt = rope_params.get("rope_type", rope_params.get("type"))
            scaling = None if rt in (None, "default") else rope_params
        if scaling is not None and scaling.get("rope_type", scaling.get("type", "default")) != "default":
            raise ModelConfigError(f"rope_scaling {scaling!r} is not supported: only unscaled rotary frequencies are")
        eps = float(d.get("rms_norm_eps", 1e-6))
        if d.get("attention_bias", False):
            raise ModelConfigError("attention_bias=true is not supported: this architecture has no bias tensors")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ModelConfigError(f"hidden_act {act!r} is not supported: the feed-forward is SwiGLU ('silu')")
        # window: layer_types wins if given; else the older trio of keys decides
        window = d.get("sliding_window")
        use_window = bool(d.get("use_sliding_window", False))
        layer_types = d.get("layer_types")
        if layer_types is None:
            first_window_layer = int(d.get("max_window_layers", layers))
            layer_types = [
                SLIDING_ATTENTION if (use_window and window is not None and i >= first_window_layer) else FULL_ATTENTION
                for i in range(layers)
            ]
        layer_types = tuple(layer_types)
        if len(layer_types) != layers:
            raise ModelConfigError(f"layer_types has {len(layer_types)} entries for {layers} layers")
        for t in layer_types:
            if t not in (FULL_ATTENTION, SLIDING_ATTENTION):
                raise ModelConfigError(f"unknown layer type {t!r}")
        if SLIDING_ATTENTION in layer_types:
            if window is None or isinstance(window, bool) or not isinstance(window, int) or window < 1:
                raise ModelConfigError("a layer is 'sliding_attention' but sliding_window is not a positive integer")
        else:
            window = None
        cfg = cls(
            architecture=archs[0],
            vocab_size=_need(d, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=_need(d, "intermediate_size", int),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rope_theta=theta,
            rms_norm_eps=eps,
            max_position_embeddings=_need(d, "max_position_embeddings", int),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            hidden_act=act,
            attention_bias=False,
            sliding_window=window,
            layer_types=layer_types,
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "Qwen3Config":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ModelConfigError("num_attention_heads must be divisible by num_key_value_heads")
        if self.head_dim < 2 or self.head_dim % 2:
            raise ModelConfigError("head_dim must be even (the rotation pairs its halves)")
        for name in ("rope_theta", "rms_norm_eps"):
            v = getattr(self, name)
            if not math.isfinite(v) or v <= 0:
                raise ModelConfigError(f"{name} must be finite and positive, got {v!r}")
        for name in ("vocab_size", "intermediate_size", "max_position_embeddings"):
            if getattr(self, name) < 1:
                raise ModelConfigError(f"{name} must be positive")

    def to_dict(self) -> dict:
        """The config.json content that reads back as this configuration."""
        d = asdict(self)
        d["architectures"] = [d.pop("architecture")]
        d["layer_types"] = list(self.layer_types)
        d["use_sliding_window"] = self.sliding_window is not None
        d["model_type"] = "qwen3"
        return d
