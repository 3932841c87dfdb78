"""Rotary position encoding."""
from __future__ import annotations

import torch

from ..config.specs import RotarySpec
from ..errors import ModelConfigError
from .registry import register_part


class Rotary:
    """inv_freq_i = 1 / theta^(2i / rotary_dim), angle = position * inv_freq_i, both in
    float32 (src/infurnace/executor/tinygrad/model.py:18-22); the rotation itself runs
    inside the attention part's fused kernel, which takes the frequencies, the rotated
    width and the pairing as arguments (model.py:24-27 is the half-split pairing)."""

    graph_safe = True     # launches depend on the step's sizes only, never on values read on the host

    def __init__(self, spec: RotarySpec, weights, runtime):
        if spec.rotary_dim % 2 or not 0 < spec.rotary_dim <= spec.head_dim:
            raise ModelConfigError(f"rotary_dim {spec.rotary_dim} must be even and at most head_dim {spec.head_dim}")
        self.spec = spec
        self.k = runtime.kernels
        exponent = torch.arange(0, spec.rotary_dim, 2, dtype=torch.float32) / spec.rotary_dim
        self.inv_freq = (1.0 / (spec.theta ** exponent)).to(runtime.device)

    def fused_rotary(self):
        return self.inv_freq, self.spec.rotary_dim, self.spec.interleaved

    def table(self, ctx):
        """(cos, sin) of every token's angles, computed once per step and shared by all layers with the same
        base and rotated width (the angles do not depend on the layer)."""
        key = ("rope_table", self.spec.theta, self.spec.rotary_dim)
        t = ctx.shared.get(key)
        if t is None:
            t = ctx.buffer(f"rope_table_{self.spec.theta}_{self.spec.rotary_dim}", (ctx.num_tokens, self.spec.rotary_dim),
                           torch.float32)
            self.k.rope_table(ctx.positions, self.inv_freq, t)
            ctx.shared[key] = t
        return t

    def apply(self, qkv, num_heads, num_kv_heads, head_dim, positions):
        self.k.qk_norm_rope_store(qkv, num_heads, num_kv_heads, head_dim, None, None, 0.0,
                                  self.inv_freq, self.spec.rotary_dim, self.spec.interleaved,
                                  positions, None, None)


register_part(RotarySpec, Rotary)
