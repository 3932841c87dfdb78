"""Embedding, LM head, and the decoder that runs the layers in the schedule's order."""
from __future__ import annotations

import torch

from ..config.specs import EmbeddingSpec, LMHeadSpec, ModelPlan
from .registry import build_part, register_part


class Embedding:
    """x[t] = table[id_t], widened to float32, no scaling
    (src/infurnace/executor/tinygrad/model.py:95)."""

    def __init__(self, spec: EmbeddingSpec, weights, runtime):
        self.spec = spec
        self.table = weights[spec.weight]
        self.k = runtime.kernels

    def forward(self, ids, out):
        self.k.embed(self.table, ids, out)
        return out


class LMHead:
    """logits = h @ W^T in float32 (model.py:151); W is the embedding table when tied
    (src/infurnace/executor/tinygrad/weights.py:68), read in place."""

    def __init__(self, spec: LMHeadSpec, weights, runtime):
        self.spec = spec
        self.weight = weights[spec.weight]
        self.k = runtime.kernels

    def forward(self, h, out):
        self.k.linear(h, self.weight, out)
        return out


register_part(EmbeddingSpec, Embedding)
register_part(LMHeadSpec, LMHead)


class DecoderModel:
    """The parts of a :class:`ModelPlan`, built once, and ``forward(ctx)``: the tokens of
    one step through every layer call of the schedule, then the final norm and the head on
    the rows whose logits are wanted (model.py:150-151 does so for the last row)."""

    def __init__(self, plan: ModelPlan, weights, runtime):
        self.plan = plan
        self.rt = runtime
        self.embedding = build_part(plan.embedding, weights, runtime)
        self.layers = [build_part(spec, weights, runtime) for spec in plan.layers]
        self.schedule = plan.resolved_schedule()
        self.final_norm = build_part(plan.final_norm, weights, runtime)
        self.lm_head = build_part(plan.lm_head, weights, runtime)

    @property
    def graph_safe(self) -> bool:
        """True when every layer's launches depend only on the sizes of a step, so that a
        decode step may be recorded once and replayed (a part says so with ``graph_safe``)."""
        return all(getattr(layer, "graph_safe", False) for layer in self.layers)

    def forward(self, ctx):
        n = ctx.num_tokens
        x = ctx.buffer("x", (n, self.plan.hidden_size), torch.float32)
        self.embedding.forward(ctx.token_ids, x)
        pending = None
        for i, call in enumerate(self.schedule):
            layer = self.layers[call.layer]
            nxt = self.layers[self.schedule[i + 1].layer] if i + 1 < len(self.schedule) else None
            if getattr(layer, "folds_norms", False) and getattr(nxt, "folds_norms", False):
                pending = layer.forward(x, pending, ctx, call, next_layer=nxt)     # may hand over a folded norm
            else:
                pending = layer.forward(x, pending, ctx, call)
        m = ctx.num_logit_rows
        if m == 0:
            return None
        hn = ctx.buffer("h_final", (m, self.plan.hidden_size), self.rt.act_dtype, rows=m)
        self.final_norm.forward(x, hn, delta=pending, rows=ctx.logit_rows)
        logits = ctx.buffer("logits", (m, self.plan.vocab_size), torch.float32, rows=m)
        self.lm_head.forward(hn, logits)
        return logits
