"""Architectures known to the engine.  Importing this package registers them; it needs
neither torch nor CUDA."""
from .registry import (  # noqa: F401
    Architecture, register_architecture, get_architecture, known_architectures,
    config_from_dict, read_config, plan_for,
)
from . import qwen3  # noqa: F401  (registers "Qwen3ForCausalLM")
