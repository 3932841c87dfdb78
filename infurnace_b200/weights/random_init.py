"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration and
a seed, or the same tensors made on the device without a folder.

The reference has no random weights; its tests build toy weights by hand
(tests/test_cached_forward.py:51-74).  Here matrices and the embedding are drawn from
N(0, 0.02) and norm weights from 1 + N(0, 0.1).  The values are counter-based: element i of a
tensor is a pure function of (seed, tensor name, i), so a tensor does not depend on which other
tensors the model has, in which order they are made, or where: :func:`normal_values` (numpy, for
the folder writer) and the kernel behind ``kernels.random_normal`` (for models too large to pass
through a file: the 8B and 32B shapes of the benchmarks) give the same bits.

The standard normal is the sum of twelve uniform 16-bit integers, centred and scaled by 2^-16
(variance 1, range +-6), taken from three words of a 64-bit mixer at counters 3i, 3i+1, 3i+2:
integer arithmetic, one exact scaling, one rounded multiply and one rounded addition in float32.
"""
from __future__ import annotations

import hashlib
import json
import os
import weakref
from collections.abc import Mapping
from typing import Optional

from ..models.registry import plan_for
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.1
_GOLDEN = 0x9E3779B97F4A7C15


def tensor_seed(seed: int, name: str) -> int:
    """64 bits that stand for (seed, tensor name)."""
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little")


def moments(shape):
    """(mean, std) of a tensor of this shape: a vector is a norm weight, anything else a matrix."""
    return (1.0, NORM_STD) if len(shape) == 1 else (0.0, MATRIX_STD)


def _signed(x: int) -> int:
    x &= (1 << 64) - 1
    return x - (1 << 64) if x >= (1 << 63) else x


def _lsr(z, k: int):
    """Logical shift right of int64 tensors (torch's ``>>`` keeps the sign)."""
    return (z >> k) & ((1 << (64 - k)) - 1)


def normal_values(seed64: int, n: int, mean: float, std: float):
    """float32 CPU tensor of n values, element i = mean + std * z_i (see the module's header).  64-bit
    integer arithmetic wraps in torch as it does on the device."""
    import torch
    gold, m1, m2 = _signed(_GOLDEN), _signed(0xBF58476D1CE4E5B9), _signed(0x94D049BB133111EB)
    out = torch.empty(n, dtype=torch.float32)
    mean_t, std_t = torch.tensor(mean, dtype=torch.float32), torch.tensor(std, dtype=torch.float32)
    chunk = 1 << 22
    for a in range(0, n, chunk):
        i3 = torch.arange(a, min(n, a + chunk), dtype=torch.int64) * 3
        total = torch.zeros_like(i3)
        for j in range(3):
            z = (i3 + j) * gold + _signed(seed64)
            z = (z ^ _lsr(z, 30)) * m1
            z = (z ^ _lsr(z, 27)) * m2
            z = z ^ _lsr(z, 31)
            total += (z & 0xFFFF) + (_lsr(z, 16) & 0xFFFF) + (_lsr(z, 32) & 0xFFFF) + _lsr(z, 48)
        zf = (total - 393210).to(torch.float32) * (1.0 / 65536.0)
        out[a:a + i3.numel()] = mean_t + std_t * zf
    return out


class _Producer:
    """Makes one tensor when called; knows shape and dtype beforehand."""

    def __init__(self, seed, name, shape, dtype, kernels=None):
        self.seed, self.name, self.shape, self.dtype, self.kernels = seed, name, tuple(shape), dtype, kernels

    def __call__(self):
        import torch
        n = 1
        for s in self.shape:
            n *= s
        mean, std = moments(self.shape)
        if self.kernels is not None:       # made on the device (the same bits), for folders of large models
            t = torch.empty(self.shape, dtype=self.dtype, device="cuda")
            self.kernels.random_normal(t, tensor_seed(self.seed, self.name), mean, std)
            return t.cpu()
        return normal_values(tensor_seed(self.seed, self.name), n, mean, std).view(self.shape).to(self.dtype)


class DeviceRandomWeights(Mapping):
    """The tensors of a plan, made on the device when asked for: ``weights[name]`` draws the tensor with
    the kernel set's ``random_normal`` in the dtype the loader would give it.  Nothing is kept beyond a
    weak reference, so a tensor that a part copies into a fused matrix and drops is freed at once, while
    a tensor that two parts read (a tied embedding) is made once as long as one of them holds it."""

    def __init__(self, plan, seed: int, engine_dtype, device, kernels, store_dtype=None, norm_dtype=None):
        """``store_dtype`` / ``norm_dtype``: the dtypes a folder of this model would store matrices and
        norm weights in (default bfloat16); values are drawn in these and then follow the loader's dtype
        policy for ``engine_dtype``, so the tensors equal those of ``write_random_model`` + ``load_weights``."""
        import torch
        self._specs = dict(plan.tensors())
        self._seed, self._engine_dtype = seed, engine_dtype
        self._store = store_dtype or torch.bfloat16
        self._norm_store = norm_dtype or self._store
        self._device, self._k = device, kernels
        self._alive = {}

    def __iter__(self):
        return iter(self._specs)

    def __len__(self):
        return len(self._specs)

    def __getitem__(self, name):
        import torch
        spec = self._specs[name]
        held = self._alive.get(name)
        t = held() if held is not None else None
        if t is None:
            if spec.kind == "int":
                raise NotImplementedError("random integer tables")
            from .loader import target_dtype
            mean, std = moments(spec.shape)
            stored = self._norm_store if len(spec.shape) == 1 else self._store
            t = torch.empty(tuple(spec.shape), dtype=stored, device=self._device)
            self._k.random_normal(t, tensor_seed(self._seed, name), mean, std)
            tag = "F32" if stored == torch.float32 else "BF16"
            t = t.to(target_dtype(tag, spec.kind, self._engine_dtype))
            self._alive[name] = weakref.ref(t)
        return t


def write_random_model(config, seed: int, out_dir: str, store_dtype: str = "bfloat16",
                       norm_dtype: Optional[str] = None, kernels=None) -> str:
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors`` for ``config``.

    ``store_dtype`` is the dtype matrices are stored in ("bfloat16" or "float32");
    ``norm_dtype`` that of the norm weights (default: the same).  ``kernels``: a CUDA kernel
    set; the tensors are then drawn on the device (the same values, much faster for large models)."""
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
        items.append((name, _Producer(seed, name, spec.shape, norm_dt if len(spec.shape) == 1 else mat_dt, kernels)))
    write_safetensors(os.path.join(out_dir, "model.safetensors"), items,
                      metadata={"format": "pt", "seed": str(seed)})
    return out_dir
