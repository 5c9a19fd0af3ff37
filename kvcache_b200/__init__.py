"""kvcache_b200: a small, whole inference engine for one GPU (NVIDIA B200, sm_100a)."""
from . import models  # registers the architectures  # noqa: F401
from .config import EngineOptions, load_config
from .engine import LLM
from .sampling import SamplingParams

__version__ = "0.1.0"
__all__ = ["EngineOptions", "load_config", "LLM", "SamplingParams"]
