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


@dataclass
class Runtime:
    """What every part is built with: the device, the dtype of activations between
    kernels (bfloat16 or float32; the residual stream and the logits are float32 in
    both), and the kernel set."""
    device: Any
    act_dtype: Any
    kernels: Any
