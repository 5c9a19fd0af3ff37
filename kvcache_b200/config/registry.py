"""One registry from an architecture's name (config.json `architectures[0]`) to its model.

An entry is a configuration class and a builder `build(config, options) -> DecoderModel`
(see `kvcache_b200.parts.model`).  The reference has no such table: its two apps
are one model each (apps/qwen_serve.cu, apps/qwen_infer.cu).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Type

from .base import ConfigError, ModelConfig, architecture_name, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Type[ModelConfig]
    build: Callable[..., Any]


_REGISTRY: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Type[ModelConfig], build: Callable[..., Any],
                          replace: bool = False) -> None:
    if name in _REGISTRY and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _REGISTRY[name] = Architecture(name, config_class, build)


def unregister_architecture(name: str) -> None:
    _REGISTRY.pop(name, None)


def registered_architectures() -> tuple:
    return tuple(sorted(_REGISTRY))


def lookup_architecture(name: str) -> Architecture:
    try:
        return _REGISTRY[name]
    except KeyError:
        known = ", ".join(registered_architectures()) or "none"
        raise ConfigError(f"unknown architecture '{name}' (registered: {known})") from None


def config_from_dict(data: Mapping[str, Any], where: str = "config.json") -> ModelConfig:
    arch = lookup_architecture(architecture_name(data, where))
    return arch.config_class.from_dict(data, where)


def load_config(folder: str) -> ModelConfig:
    """Reads `<folder>/config.json` into the typed configuration of its architecture."""
    import os
    return config_from_dict(read_config_json(folder), os.path.join(folder, "config.json"))
