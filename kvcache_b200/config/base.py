"""Typed model configuration: the base class and the helpers that read config.json keys.

The reference keeps every model size as a compile-time constant
(apps/qwen_serve.cu:20-23) and writes, but never reads, a config block
(tools/dump_weights.py:46-58).  Here the sizes come from the architecture's own
config.json and nowhere else.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Any, Dict, Mapping, Optional, Sequence, Tuple


class ConfigError(ValueError):
    """A config.json that cannot describe a model this engine can build."""


_MISSING = object()


class KeyReader:
    """Reads keys of a config.json mapping and collects every problem before raising."""

    def __init__(self, data: Mapping[str, Any], where: str = "config.json"):
        self.data = data
        self.where = where
        self.problems: list[str] = []

    def _get(self, key: str, default: Any = _MISSING) -> Any:
        value = self.data.get(key, _MISSING)
        if value is _MISSING or value is None:
            if default is _MISSING:
                self.problems.append(f"missing key '{key}'")
                return None
            return default
        return value

    def integer(self, key: str, default: Any = _MISSING, minimum: Optional[int] = None) -> Optional[int]:
        value = self._get(key, default)
        if value is None:
            return None
        if isinstance(value, bool) or not isinstance(value, int):
            if isinstance(value, float) and value == int(value):
                value = int(value)
            else:
                self.problems.append(f"'{key}' must be an integer, got {value!r}")
                return None
        if minimum is not None and value < minimum:
            self.problems.append(f"'{key}' must be >= {minimum}, got {value}")
        return value

    def number(self, key: str, default: Any = _MISSING, positive: bool = False) -> Optional[float]:
        value = self._get(key, default)
        if value is None:
            return None
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            self.problems.append(f"'{key}' must be a number, got {value!r}")
            return None
        value = float(value)
        if positive and not value > 0.0:
            self.problems.append(f"'{key}' must be > 0, got {value}")
        return value

    def boolean(self, key: str, default: Any = _MISSING) -> Optional[bool]:
        value = self._get(key, default)
        if value is None:
            return None
        if not isinstance(value, bool):
            self.problems.append(f"'{key}' must be true or false, got {value!r}")
            return None
        return value

    def string(self, key: str, default: Any = _MISSING) -> Optional[str]:
        value = self._get(key, default)
        if value is None:
            return None
        if not isinstance(value, str):
            self.problems.append(f"'{key}' must be a string, got {value!r}")
            return None
        return value

    def int_list(self, key: str, default: Any = _MISSING) -> Optional[Tuple[int, ...]]:
        """An integer or a list of integers (eos_token_id comes in both forms)."""
        value = self._get(key, default)
        if value is None:
            return None
        if isinstance(value, int) and not isinstance(value, bool):
            return (value,)
        if isinstance(value, (list, tuple)) and all(isinstance(v, int) and not isinstance(v, bool) for v in value):
            return tuple(value)
        self.problems.append(f"'{key}' must be an integer or a list of integers, got {value!r}")
        return None

    def fail(self, message: str) -> None:
        self.problems.append(message)

    def finish(self) -> None:
        if self.problems:
            raise ConfigError(f"{self.where}: " + "; ".join(self.problems))


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration.

    Subclasses are frozen dataclasses whose fields mirror the architecture's
    config.json keys; `from_dict` validates, `to_dict` writes the same keys back
    so that a random-weights folder round-trips.
    """

    architecture: str

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str = "config.json") -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        raise NotImplementedError

    def replace(self, **changes: Any) -> "ModelConfig":
        current = {f.name: getattr(self, f.name) for f in fields(self)}
        current.update(changes)
        return type(self)(**current)


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no such file (a model folder holds config.json and model.safetensors)")
    with open(path, "r", encoding="utf-8") as fh:
        try:
            data = json.load(fh)
        except json.JSONDecodeError as exc:
            raise ConfigError(f"{path}: not valid JSON ({exc})") from None
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return data


def architecture_name(data: Mapping[str, Any], where: str = "config.json") -> str:
    archs = data.get("architectures")
    if not isinstance(archs, Sequence) or isinstance(archs, str) or len(archs) == 0 or not isinstance(archs[0], str):
        raise ConfigError(f"{where}: 'architectures' must be a non-empty list of names")
    return archs[0]
