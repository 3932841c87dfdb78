"""How a layer's parts are arranged."""
from __future__ import annotations

from ..config.specs import PreNormBlockSpec
from .registry import Folded, build_part, register_part


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

    folds_norms = True

    def takes_folded(self, n):
        """Whether the block before this one may hand over x already updated and this block's
        first norm folded (a :class:`Folded` as ``pending``) for a step of n tokens."""
        take = getattr(self.mixer, "can_take_folded", None)
        return bool(getattr(self.mixer_norm, "foldable", False) and take and take(n))

    def forward(self, x, pending, ctx, call, next_layer=None):
        n = x.shape[0]
        if isinstance(pending, Folded):              # x is up to date and our first norm is folded
            h = pending
        else:
            h = ctx.buffer("h", x.shape, self.rt.act_dtype)
            self.mixer_norm.forward(x, h, delta=pending)
        take = getattr(self.ffn, "can_take_folded", None)
        if getattr(self.mixer, "can_fold_output", False) and getattr(self.ffn_norm, "foldable", False) and take and take(n):
            d = self.mixer.forward(h, ctx, call, fold=(x, self.ffn_norm))
        else:
            d = self.mixer.forward(h, ctx, call)
        if isinstance(d, Folded):
            h = d
        else:
            h = ctx.buffer("h", x.shape, self.rt.act_dtype)
            self.ffn_norm.forward(x, h, delta=d)
        if next_layer is not None and getattr(self.ffn, "can_fold_output", False) and next_layer.takes_folded(n):
            return self.ffn.forward(h, ctx, fold=(x, next_layer.mixer_norm))
        return self.ffn.forward(h, ctx)


register_part(PreNormBlockSpec, PreNormBlock)
