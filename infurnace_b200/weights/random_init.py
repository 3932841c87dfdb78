"""Random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed.

The reference has no random weights; its tests build toy weights by hand
(tests/test_cached_forward.py:51-74).  Here matrices and the embedding are drawn from
N(0, 0.02) and norm weights from 1 + N(0, 0.1).  Each tensor has a generator of its own,
seeded from (seed, tensor name), so the values of a tensor do not depend on which other
tensors the model has or in which order they are written.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Optional

from ..models.registry import plan_for
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.1


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


class _Producer:
    """Makes one tensor when called; knows shape and dtype beforehand."""

    def __init__(self, seed, name, shape, dtype):
        self.seed, self.name, self.shape, self.dtype = seed, name, tuple(shape), dtype

    def __call__(self):
        import torch
        g = torch.Generator(device="cpu")
        g.manual_seed(_tensor_seed(self.seed, self.name))
        x = torch.randn(self.shape, generator=g, dtype=torch.float32)
        if len(self.shape) == 1:            # a norm weight
            x = 1.0 + NORM_STD * x
        else:
            x = MATRIX_STD * x
        return x.to(self.dtype)


def write_random_model(config, seed: int, out_dir: str, store_dtype: str = "bfloat16",
                       norm_dtype: Optional[str] = None) -> str:
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors`` for ``config``.

    ``store_dtype`` is the dtype matrices are stored in ("bfloat16" or "float32");
    ``norm_dtype`` that of the norm weights (default: the same)."""
    import torch
    plan = plan_for(config)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=1)
    mat_dt = getattr(torch, store_dtype)
    norm_dt = getattr(torch, norm_dtype or store_dtype)
    items = []
    for name, spec in plan.tensors().items():
        if spec.kind == "int":
            raise NotImplementedError("random integer tables")
        items.append((name, _Producer(seed, name, spec.shape, norm_dt if len(spec.shape) == 1 else mat_dt)))
    write_safetensors(os.path.join(out_dir, "model.safetensors"), items,
                      metadata={"format": "pt", "seed": str(seed)})
    return out_dir
