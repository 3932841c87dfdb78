"""From a part's description to the class that runs it.

``register_part(SpecType, ImplClass)`` ties a description type
(infurnace_b200/config/specs.py, or one defined elsewhere) to its implementation;
``build_part(spec, weights, runtime)`` makes the object.  An implementation's
constructor takes ``(spec, weights, runtime)``: the description, a mapping from tensor
name to device tensor, and the :class:`Runtime`.  No implementation knows which model
it is in: it sees its own description and the tensors that description names.

Interfaces, by role:

* norm:            ``forward(x, out, delta=None, rows=None)``  (x: float32 residual stream)
* position code:   ``fused_rotary() -> (inv_freq, rotary_dim, interleaved) | None`` and
                   ``apply(qkv, num_heads, num_kv_heads, head_dim, positions)``
* mixer:           ``forward(h, ctx, call) -> delta``  (float32 [N, H] or [S, N, H])
* feed-forward:    ``forward(h, ctx) -> delta``
* block:           ``forward(x, pending, ctx, call) -> pending``; the block adds
                   ``pending`` (the previous block's last delta) to x before its first norm
                   and returns its own last delta instead of adding it
* embedding:       ``forward(ids, out)``;  LM head: ``forward(h, out)``

A norm folded into its neighbours (optional; a part without these attributes is simply
given plain tensors and asked for plain deltas).  RMSNorm(v) = v * g * r with one number r
per row, so the product that makes v can write v * g and partial sums of v^2, and the
product that reads it can multiply its rows by r at the end: no kernel runs for the norm.

* a norm with ``foldable = True`` exposes ``weight`` and ``spec.eps``;
* a mixer or feed-forward with ``can_fold_output = True`` takes ``fold=(x, norm)`` and may
  then add its result to x itself and return a :class:`Folded` for ``norm`` instead of a delta;
* one with ``can_take_folded(n)`` true accepts a :class:`Folded` as ``h``;
* a block with ``folds_norms = True`` takes ``next_layer=`` (the block that runs after it),
  offers ``takes_folded(n)`` and accepts a :class:`Folded` as ``pending``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict

_PARTS: Dict[type, Any] = {}


def register_part(spec_type: type, impl, *, replace: bool = False) -> None:
    if spec_type in _PARTS and not replace:
        raise ValueError(f"a part is already registered for {spec_type.__name__}")
    _PARTS[spec_type] = impl


def build_part(spec, weights, runtime):
    try:
        impl = _PARTS[type(spec)]
    except KeyError:
        raise KeyError(f"no part registered for description type {type(spec).__name__}") from None
    return impl(spec, weights, runtime)


class Folded:
    """An activation whose RMSNorm is half done: ``values`` holds v * g in the activation
    dtype and ``row_scale`` = (partials, parts, eps, width) is what a product needs to
    finish it (``kernels.linear(..., row_scale=...)``)."""
    __slots__ = ("values", "row_scale")

    def __init__(self, values, row_scale):
        self.values = values
        self.row_scale = row_scale

    @property
    def shape(self):
        return self.values.shape


def unfolded(h):
    """(tensor, row_scale or None) of a plain tensor or a :class:`Folded`."""
    return (h.values, h.row_scale) if isinstance(h, Folded) else (h, None)


def fold_residual_norm(kernels, ctx, tag, a, w, fold, act_dtype):
    """The last product of a mixer or feed-forward with the residual addition and the next
    norm folded in, if the kernels can do it for these sizes: returns a :class:`Folded`,
    or None (then the caller runs the plain product).  ``fold`` = (x, norm)."""
    if fold is None or not getattr(kernels, "can_fold_norm", None):
        return None
    x, norm = fold
    n, o = a.shape[0], w.shape[0]
    if a.dtype != act_dtype or x.shape != (n, o) or not kernels.can_fold_norm(n, a.dtype, w):
        return None
    parts = kernels.fold_parts(o, n, w)
    out = ctx.buffer("folded_" + tag, (n, o), act_dtype)
    # one flat buffer whatever the number of rows, so that its address stays the same from step to step
    partials = ctx.buffer("folded_partials_" + tag, (parts * n,), __import__("torch").float32).view(parts, n)
    kernels.linear_residual_norm(a, w, x, norm.weight, out, partials)
    return Folded(out, (partials, parts, float(norm.spec.eps), o))


@dataclass
class Runtime:
    """What every part is built with: the device, the dtype of activations between
    kernels (bfloat16 or float32; the residual stream and the logits are float32 in
    both), and the kernel set."""
    device: Any
    act_dtype: Any
    kernels: Any
