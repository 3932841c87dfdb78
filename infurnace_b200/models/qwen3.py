"""Qwen3 dense: the plan builder (configuration -> layers, order, tensor names).

Layer order and formulas follow src/infurnace/executor/tinygrad/model.py:98-151: a
pre-norm decoder whose every block is RMSNorm -> grouped-query attention with
per-head RMSNorm of q and k before half-split rotary encoding -> residual -> RMSNorm
-> SwiGLU feed-forward -> residual; then a final RMSNorm and an LM head that is tied
to the embedding or a tensor of its own.  Tensor names are those of the safetensors
checkpoints of this architecture; the reference's GGUF names for the same tensors are
listed in src/infurnace/models/qwen3.py:41-59.
"""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config, SLIDING_ATTENTION
from ..config.specs import (
    AttentionSpec, EmbeddingSpec, GatedMLPSpec, LayerCall, LMHeadSpec, ModelPlan,
    PreNormBlockSpec, RMSNormSpec, RotarySpec,
)
from .registry import register_architecture


def build_qwen3_plan(cfg: Qwen3Config) -> ModelPlan:
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        window = cfg.sliding_window if cfg.layer_types[i] == SLIDING_ATTENTION else None
        attn = AttentionSpec(
            hidden_size=cfg.hidden_size,
            num_heads=cfg.num_attention_heads,
            num_kv_heads=cfg.num_key_value_heads,
            head_dim=cfg.head_dim,
            scale=cfg.head_dim ** -0.5,
            q_proj=f"{p}.self_attn.q_proj.weight",
            k_proj=f"{p}.self_attn.k_proj.weight",
            v_proj=f"{p}.self_attn.v_proj.weight",
            o_proj=f"{p}.self_attn.o_proj.weight",
            q_norm=RMSNormSpec(cfg.head_dim, cfg.rms_norm_eps, f"{p}.self_attn.q_norm.weight"),
            k_norm=RMSNormSpec(cfg.head_dim, cfg.rms_norm_eps, f"{p}.self_attn.k_norm.weight"),
            position=RotarySpec(cfg.head_dim, cfg.head_dim, cfg.rope_theta, interleaved=False),
            window=window,
        )
        mlp = GatedMLPSpec(
            hidden_size=cfg.hidden_size,
            intermediate_size=cfg.intermediate_size,
            activation=cfg.hidden_act,
            gate_proj=f"{p}.mlp.gate_proj.weight",
            up_proj=f"{p}.mlp.up_proj.weight",
            down_proj=f"{p}.mlp.down_proj.weight",
        )
        layers.append(PreNormBlockSpec(
            mixer_norm=RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps, f"{p}.input_layernorm.weight"),
            mixer=attn,
            ffn_norm=RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps, f"{p}.post_attention_layernorm.weight"),
            ffn=mlp,
        ))
    embed_name = "model.embed_tokens.weight"
    return ModelPlan(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        max_positions=cfg.max_position_embeddings,
        embedding=EmbeddingSpec(cfg.vocab_size, cfg.hidden_size, embed_name),
        layers=tuple(layers),
        schedule=tuple(LayerCall(i) for i in range(cfg.num_hidden_layers)),
        final_norm=RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps, "model.norm.weight"),
        lm_head=LMHeadSpec(cfg.vocab_size, cfg.hidden_size,
                           embed_name if cfg.tie_word_embeddings else "lm_head.weight",
                           tied=cfg.tie_word_embeddings, stored_as="lm_head.weight"),
    )


register_architecture("Qwen3ForCausalLM", Qwen3Config, build_qwen3_plan)
