"""One registry from an architecture's name (config.json `architectures[0]`) to its typed
configuration and to the builder that lays the model out as a `ModelSpec`.

cuongvng/bare-cuda-4gib has a single hard-wired model (engine/src/model.cpp); the registry is
what lets another architecture be added here without touching the engine: write a config class
with `from_dict`, a function config -> ModelSpec, and call `register_architecture`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict

from ..errors import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type                      # has from_dict(dict) and to_dict()
    build_spec: Callable[[Any], Any]        # config -> parts.spec.ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, build_spec: Callable[[Any], Any]) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_class, build_spec)


def registered_architectures():
    return sorted(_ARCHITECTURES)


def resolve_architecture(config_dict: Dict[str, Any]) -> Architecture:
    names = config_dict.get("architectures")
    if not names or not isinstance(names, (list, tuple)) or not isinstance(names[0], str):
        raise ConfigError("config.json: 'architectures' must be a list that names the model class")
    if names[0] not in _ARCHITECTURES:
        raise ConfigError(f"config.json: architecture '{names[0]}' is not registered "
                          f"(registered: {registered_architectures()})")
    return _ARCHITECTURES[names[0]]
