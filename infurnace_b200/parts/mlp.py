"""The dense gated feed-forward."""
from __future__ import annotations

import torch

from ..config.specs import GatedMLPSpec
from ..errors import ModelConfigError
from .registry import fold_residual_norm, register_part, unfolded


class GatedMLP:
    """down(silu(gate(h)) * up(h)) (src/infurnace/executor/tinygrad/model.py:146-148).
    gate and up run as one product against their row-wise concatenation (exact), with the
    activation and the product of the two halves in that kernel's epilogue."""

    graph_safe = True     # launches depend on the step's sizes only, never on values read on the host

    def __init__(self, spec: GatedMLPSpec, weights, runtime):
        if spec.activation != "silu":
            raise ModelConfigError(f"activation {spec.activation!r}: only 'silu' has a kernel")
        self.spec = spec
        self.rt = runtime
        self.k = runtime.kernels
        self.w_gate_up = torch.cat((weights[spec.gate_proj], weights[spec.up_proj]), dim=0).contiguous()
        self.w_down = weights[spec.down_proj]

    can_fold_output = True

    def can_take_folded(self, n):
        can = getattr(self.k, "can_fold_norm", None)
        return bool(can and can(n, self.rt.act_dtype, self.w_gate_up, "silu_gate"))

    def forward(self, h, ctx, fold=None):
        h, row_scale = unfolded(h)
        n = h.shape[0]
        act = ctx.buffer("ffn_act", (n, self.spec.intermediate_size), self.rt.act_dtype)
        if row_scale is not None:
            self.k.linear(h, self.w_gate_up, act, epilogue="silu_gate", row_scale=row_scale)
        else:
            self.k.linear(h, self.w_gate_up, act, epilogue="silu_gate")
        folded = fold_residual_norm(self.k, ctx, "ffn", act, self.w_down, fold, self.rt.act_dtype)
        if folded is not None:
            return folded
        delta = ctx.buffer("delta_ffn", (n, self.spec.hidden_size), torch.float32)
        self.k.linear(act, self.w_down, delta)
        return delta


register_part(GatedMLPSpec, GatedMLP)
