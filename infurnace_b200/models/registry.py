"""One registry from the architecture's name (config.json ``architectures[0]``) to its model.

The reference wires its single architecture by imports (src/infurnace/cli.py:33-36) and
says that model differences stay in the model layer (docs/architecture.md:393-402).
Here an architecture is an entry of this table: a configuration class with
``from_dict`` and a plan builder that turns the configuration into a
:class:`~infurnace_b200.config.specs.ModelPlan`.  Everything else (loader, cache
manager, step function, scheduler, replay) works from the plan.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from ..errors import ModelConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                      # has from_dict(mapping) -> config
    build_plan: Callable[[Any], Any]       # config -> ModelPlan


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class, build_plan, *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ModelConfigError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_class, build_plan)


def known_architectures():
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ModelConfigError(
            f"unknown architecture {name!r}; known: {', '.join(known_architectures()) or '(none)'}") from None


def config_from_dict(d: Mapping[str, Any]):
    archs = d.get("architectures") if isinstance(d, Mapping) else None
    if not isinstance(archs, (list, tuple)) or not archs:
        raise ModelConfigError("config.json lacks required key 'architectures'")
    return get_architecture(archs[0]).config_class.from_dict(d)


def read_config(model_dir: str):
    """The typed configuration of the model folder (or config file) at ``model_dir``."""
    path = os.path.join(model_dir, "config.json") if os.path.isdir(model_dir) else model_dir
    if not os.path.exists(path):
        raise ModelConfigError(f"no config.json at {path}")
    with open(path, "r", encoding="utf-8") as f:
        return config_from_dict(json.load(f))


def plan_for(config):
    """The :class:`ModelPlan` of a configuration, through its architecture's builder."""
    return get_architecture(config.architecture).build_plan(config)
