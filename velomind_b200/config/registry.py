"""One registry from an architecture's name (config.json `architectures[0]`) to its model.

An entry holds the typed configuration class and the function that turns a
configuration into a `ModelPlan`.  The reference has no such table (the model
family is fixed at compile time, examples/smollm2/smollm2_engine.cpp:43-68);
here config.json chooses.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict

from .base import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[Dict[str, Any], str], Any]
    plan: Callable[[Any], Any]          # typed config -> parts.spec.ModelPlan


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_from_dict, plan) -> Architecture:
    """Add (or replace) an architecture.  `config_from_dict(data, where)` returns the typed
    configuration; `plan(config)` returns the `ModelPlan` the engine builds parts from."""
    arch = Architecture(name, config_from_dict, plan)
    _ARCHITECTURES[name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures():
    return sorted(_ARCHITECTURES)


def architecture_name(data: Dict[str, Any], where: str = "config.json") -> str:
    archs = data.get("architectures")
    if not isinstance(archs, list) or len(archs) == 0 or not isinstance(archs[0], str):
        raise ConfigError(f"{where}: missing required key 'architectures' (a list whose first entry names the model class)")
    return archs[0]


def resolve(data: Dict[str, Any], where: str = "config.json") -> Architecture:
    name = architecture_name(data, where)
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"{where}: architecture {name!r} is not registered; registered: {', '.join(registered_architectures()) or '(none)'}")
    return _ARCHITECTURES[name]
