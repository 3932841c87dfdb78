"""Typed errors of the engine, one per subsystem.

The reference keeps the same family (``ModelConfigError`` in
src/infurnace/models/config.py:4, ``WeightMappingError`` in
src/infurnace/executor/tinygrad/weights.py:13, ``Qwen3ModelError`` in
src/infurnace/executor/tinygrad/model.py:8, ``SchedulerError`` in
src/infurnace/scheduler/scheduler.py:8).
"""


class InfurnaceError(Exception):
    """Base class of every error this package raises on purpose."""


class ModelConfigError(InfurnaceError, ValueError):
    """config.json does not describe a model this engine can build."""


class WeightError(InfurnaceError, ValueError):
    """The weight files do not match the tensor inventory of the model."""


class CacheError(InfurnaceError, RuntimeError):
    """A page or a state slot was used against the cache manager's rules."""


class OutOfPages(CacheError):
    """An allocation asked for more pages than the pool has free; nothing was taken."""


class BatchError(InfurnaceError, ValueError):
    """A step's batch is malformed (bad positions, unknown request, too many tokens)."""


class SchedulerError(InfurnaceError, ValueError):
    """A request or a scheduler option breaks the admission or scheduling contract."""


class KernelError(InfurnaceError, RuntimeError):
    """A CUDA kernel library is missing, failed to build, or refused the sizes it was given."""
