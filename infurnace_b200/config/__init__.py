"""Typed configurations and the plain-data description of a model (no torch needed)."""
from .specs import (  # noqa: F401
    TensorSpec, KVCacheNeed, StateNeed, RMSNormSpec, RotarySpec, AttentionSpec, GatedMLPSpec,
    PreNormBlockSpec, EmbeddingSpec, LMHeadSpec, LayerCall, ModelPlan,
)
from .qwen3 import Qwen3Config  # noqa: F401
