"""CUDA kernels of the engine.  ``load_cuda_kernels()`` compiles (first use) and loads them;
it raises :class:`~infurnace_b200.errors.KernelError` when there is no CUDA device."""
from __future__ import annotations

from .build import load_library, register_library  # noqa: F401  (for parts that bring kernels of their own)

_kernels = None


def load_cuda_kernels(progress=None):
    global _kernels
    if _kernels is None:
        from .cuda import CudaKernels
        _kernels = CudaKernels(progress=progress)
    return _kernels
