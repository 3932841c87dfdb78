"""RMSNorm with the residual addition folded in."""
from __future__ import annotations

from ..config.specs import RMSNormSpec
from .registry import register_part


class RMSNorm:
    """out = (x + delta) * rsqrt(mean((x + delta)^2) + eps) * weight, statistics in 32-bit
    (src/infurnace/executor/tinygrad/model.py:11-13).  x is the float32 residual stream;
    without ``rows`` the sum is written back to x, which is the reference's ``x = x + ...``
    (model.py:143,148) done in the same pass."""

    graph_safe = True     # launches depend on the step's sizes only, never on values read on the host
    foldable = True       # weight and spec.eps are all that a neighbouring product needs to do this norm

    def __init__(self, spec: RMSNormSpec, weights, runtime):
        self.spec = spec
        self.weight = weights[spec.weight]
        self.k = runtime.kernels

    def forward(self, x, out, delta=None, rows=None):
        self.k.rmsnorm(x, self.weight, self.spec.eps, out, delta=delta, rows=rows)
        return out


register_part(RMSNormSpec, RMSNorm)
