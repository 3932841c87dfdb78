"""The parts layers are put together from.  Importing the package registers the
implementations of the descriptions in ``infurnace_b200.config.specs``."""
from .registry import Runtime, build_part, register_part  # noqa: F401
from . import norm, rotary, attention, mlp, block, model  # noqa: F401
from .model import DecoderModel  # noqa: F401
