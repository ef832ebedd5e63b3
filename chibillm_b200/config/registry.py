"""The one registry from an architecture's name to its configuration and model.

The reference dispatches on ``config.json["model_type"]`` in a switch
(src/model_factory.cc:26-40).  Here an architecture is an entry of a table
keyed by ``architectures[0]`` (with ``model_type`` as a second key), so adding
one is a call to :func:`register_architecture`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional

from .base import ConfigError, read_config_json
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    model_type: Optional[str]
    read_config: Callable[[dict], Any]        # config.json object -> typed configuration
    model_spec: Callable[[Any], ModelSpec]    # typed configuration -> parts


_BY_NAME: Dict[str, Architecture] = {}
_BY_MODEL_TYPE: Dict[str, Architecture] = {}


def register_architecture(name: str, read_config: Callable[[dict], Any],
                          model_spec: Callable[[Any], ModelSpec],
                          model_type: Optional[str] = None, replace: bool = False) -> Architecture:
    if name in _BY_NAME and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    arch = Architecture(name, model_type, read_config, model_spec)
    _BY_NAME[name] = arch
    if model_type is not None:
        _BY_MODEL_TYPE[model_type] = arch
    return arch


def unregister_architecture(name: str) -> None:
    arch = _BY_NAME.pop(name, None)
    if arch is not None and arch.model_type is not None:
        _BY_MODEL_TYPE.pop(arch.model_type, None)


def registered_architectures() -> list:
    return sorted(_BY_NAME)


def find_architecture(config_object: dict) -> Architecture:
    """Pick the architecture that a parsed config.json names."""
    names = config_object.get("architectures")
    if isinstance(names, list) and names and isinstance(names[0], str):
        if names[0] in _BY_NAME:
            return _BY_NAME[names[0]]
        raise ConfigError("unsupported_architecture",
                          f"architecture '{names[0]}' is not registered; known: {registered_architectures()}")
    model_type = config_object.get("model_type")
    if isinstance(model_type, str):
        if model_type in _BY_MODEL_TYPE:
            return _BY_MODEL_TYPE[model_type]
        raise ConfigError("unsupported_architecture",
                          f"model_type '{model_type}' is not registered; known: {sorted(_BY_MODEL_TYPE)}")
    raise ConfigError("invalid_config", "config.json names neither 'architectures' nor 'model_type'")


def load_config(model_dir: str):
    """Read ``model_dir/config.json``; returns (architecture, typed config, spec)."""
    obj = read_config_json(model_dir)
    arch = find_architecture(obj)
    config = arch.read_config(obj)
    return arch, config, arch.model_spec(config)
