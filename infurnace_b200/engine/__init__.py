"""Step function, scheduler, request life cycle and the engine loop."""
from .loading import EngineOptions, build_runner  # noqa: F401
from .request import Request, RequestMetrics, RequestState, SamplingParams  # noqa: F401
from .runner import ModelRunner, StepEntry  # noqa: F401
from .scheduler import Scheduler, StepPlan, PlannedEntry  # noqa: F401
from .engine import Engine, EngineStepResult, generate  # noqa: F401
