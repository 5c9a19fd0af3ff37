"""Architectures known to the registry; importing this package registers them."""
from . import qwen2  # noqa: F401
from .qwen2 import build_qwen2

__all__ = ["build_qwen2"]
