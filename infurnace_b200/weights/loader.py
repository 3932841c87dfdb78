"""Weights from safetensors, by tensor name, checked against the model's inventory.

The rule is the reference's (src/infurnace/executor/tinygrad/weights.py:42-55): the set
of names in the files must equal the inventory, every shape must match, and all of this
is checked before any tensor is read or converted
(tests/test_model_weights.py:80-103).  One :class:`WeightError` lists everything that is
wrong: missing tensors, unexpected tensors and wrong shapes.  One exception to "equal":
a tied model's folder may also store the head under its own name; the reference demands
that head and embedding be one object (weights.py:68, model.py:34-36), so here the stored
head is accepted if it equals the embedding table bit for bit, and is an error otherwise.

Dtypes.  In bfloat16 mode a floating tensor is kept in bfloat16, except that a tensor
stored in 32-bit stays in 32-bit (float16 is converted to bfloat16); in float32 mode
every floating tensor is widened to float32.  Integer tables become int32.
"""
from __future__ import annotations

import sys
import time
from typing import Dict, Mapping

from ..errors import WeightError
from .safetensors_io import SafetensorsFile, list_weight_files

_FLOAT_TAGS = {"F64", "F32", "F16", "BF16"}
_INT_TAGS = {"I64", "I32", "I16", "I8", "U8"}


def check_inventory(found: Mapping[str, tuple], expected: Mapping[str, "object"],
                    duplicates: Mapping[str, str] = {}) -> None:
    """``found``: name -> (dtype tag, shape).  ``duplicates``: names that may be present beside the
    inventory, each with the tensor it must copy (same shape and dtype here; the bytes are compared by
    the caller).  Raises one error naming every fault."""
    missing = sorted(set(expected) - set(found))
    unexpected = sorted(set(found) - set(expected) - set(duplicates))
    wrong = []
    for name, of in sorted(duplicates.items()):
        if name in found and of in found and tuple(found[name]) != tuple(found[of]):
            wrong.append(f"{name}: stored beside {of}, which it must equal, as {found[name][0]} {tuple(found[name][1])} "
                         f"against {found[of][0]} {tuple(found[of][1])}")
    for name in sorted(set(expected) & set(found)):
        tag, shape = found[name]
        spec = expected[name]
        if tuple(shape) != tuple(spec.shape):
            wrong.append(f"{name}: expected {tuple(spec.shape)}, got {tuple(shape)}")
        elif spec.kind == "float" and tag not in _FLOAT_TAGS:
            wrong.append(f"{name}: expected a floating dtype, got {tag}")
        elif spec.kind == "int" and tag not in _INT_TAGS:
            wrong.append(f"{name}: expected an integer dtype, got {tag}")
    if missing or unexpected or wrong:
        parts = []
        if missing:
            parts.append(f"missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            parts.append(f"unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            parts.append(f"wrong shape or dtype ({len(wrong)}): " + "; ".join(wrong))
        raise WeightError("weights do not match the model: " + " | ".join(parts))


def target_dtype(tag: str, kind: str, engine_dtype):
    import torch
    if kind == "int":
        return torch.int32
    if engine_dtype == torch.float32:
        return torch.float32
    return torch.float32 if tag in ("F32", "F64") else torch.bfloat16


def load_weights(model_dir: str, plan, engine_dtype, device, progress=None) -> Dict[str, "object"]:
    """All tensors of ``plan`` from the folder's safetensors files, on ``device``."""
    import torch
    files = [SafetensorsFile(p) for p in list_weight_files(model_dir)]
    try:
        found, owner = {}, {}
        dup = []
        for f in files:
            for name, entry in f.entries.items():
                if name in found:
                    dup.append(name)
                found[name], owner[name] = entry, f
        if dup:
            raise WeightError("tensors stored twice: " + ", ".join(sorted(dup)))
        expected = plan.tensors()
        duplicates = plan.duplicates() if hasattr(plan, "duplicates") else {}
        check_inventory(found, expected, duplicates)
        for name, of in sorted(duplicates.items()):
            if name in found:
                a, b = owner[name].tensor(name), owner[of].tensor(of)
                if not torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8)):
                    raise WeightError(f"weights do not match the model: unexpected tensors (1): {name} (the model ties it to "
                                      f"{of}, and the two differ)")
        out = {}
        last = time.monotonic()
        for i, (name, spec) in enumerate(expected.items()):
            tag, _ = found[name]
            t = owner[name].tensor(name)
            out[name] = t.to(device=device, dtype=target_dtype(tag, spec.kind, engine_dtype), copy=True)
            if progress is not None and time.monotonic() - last > 5.0:
                progress(f"loading weights: {i + 1}/{len(expected)} tensors")
                last = time.monotonic()
        return out
    finally:
        for f in files:
            f.close()
