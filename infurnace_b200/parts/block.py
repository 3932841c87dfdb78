"""How a layer's parts are arranged."""
from __future__ import annotations

from ..config.specs import PreNormBlockSpec
from .registry import build_part, register_part


class PreNormBlock:
    """x += mixer(norm(x)); x += ffn(norm(x))
    (src/infurnace/executor/tinygrad/model.py:101,143,145,148).  Each addition happens in
    the kernel of the norm that follows it, so the block takes the previous block's last
    delta as ``pending`` and hands its own on."""

    def __init__(self, spec: PreNormBlockSpec, weights, runtime):
        self.spec = spec
        self.rt = runtime
        self.mixer_norm = build_part(spec.mixer_norm, weights, runtime)
        self.mixer = build_part(spec.mixer, weights, runtime)
        self.ffn_norm = build_part(spec.ffn_norm, weights, runtime)
        self.ffn = build_part(spec.ffn, weights, runtime)

    @property
    def graph_safe(self):
        return all(getattr(p, "graph_safe", False) for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn))

    def forward(self, x, pending, ctx, call):
        h = ctx.buffer("h", x.shape, self.rt.act_dtype)
        self.mixer_norm.forward(x, h, delta=pending)
        d = self.mixer.forward(h, ctx, call)
        self.ffn_norm.forward(x, h, delta=d)
        return self.ffn.forward(h, ctx)


register_part(PreNormBlockSpec, PreNormBlock)
