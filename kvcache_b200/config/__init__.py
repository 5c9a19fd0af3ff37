from .base import ConfigError, ModelConfig, read_config_json, architecture_name
from .options import EngineOptions, canonical_dtype
from .qwen2 import Qwen2Config, QWEN2_ARCHITECTURE
from .registry import (Architecture, config_from_dict, load_config, lookup_architecture,
                       register_architecture, registered_architectures, unregister_architecture)

__all__ = [
    "ConfigError", "ModelConfig", "read_config_json", "architecture_name", "EngineOptions",
    "canonical_dtype", "Qwen2Config", "QWEN2_ARCHITECTURE", "Architecture", "config_from_dict",
    "load_config", "lookup_architecture", "register_architecture", "registered_architectures",
    "unregister_architecture",
]
