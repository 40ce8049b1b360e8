"""One registry from an architecture's name (``config.json["architectures"][0]``) to its typed
configuration and its model class.  The reference selects a loader per model family from an enum
(model/ModelType.java:24-75 of the reference project, unknown names throw at :66-71); here a name
maps to data, and tests may register further architectures without touching the package."""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Callable

from .base import ConfigError, ModelConfig, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    model_factory: Callable  # (config, dtype, device) -> model; resolved lazily to keep config import light


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, model_factory: Callable | None = None, *,
                          replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture {name!r} is already registered")
    if model_factory is None:
        def model_factory(config, dtype, device):  # the generic decoder assembled from parts
            from ..engine.model import CausalLM
            return CausalLM(config, dtype=dtype, device=device)
    _ARCHITECTURES[name] = Architecture(name, config_class, model_factory)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_of(config_dict: dict) -> Architecture:
    archs = config_dict.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError('config.json needs "architectures": ["<name>"]')
    name = archs[0]
    arch = _ARCHITECTURES.get(name)
    if arch is None:
        raise ConfigError(f"unknown architecture {name!r}; registered: {', '.join(registered_architectures()) or 'none'}")
    return arch


def config_from_dict(config_dict: dict) -> ModelConfig:
    return architecture_of(config_dict).config_class.from_dict(config_dict)


def load_config(model_dir: str | Path) -> ModelConfig:
    return config_from_dict(read_config_json(model_dir))
