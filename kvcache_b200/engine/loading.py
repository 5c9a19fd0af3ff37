"""From a model folder to a model on the device: config.json picks the architecture from the
registry, the architecture's builder puts the parts together, and the loader hands each part
its tensors by name (replacing src/include/qwen_loader.h:27-74)."""
from __future__ import annotations

from typing import Optional

import torch

from ..config.options import canonical_dtype
from ..config.registry import load_config, lookup_architecture
from ..parts.model import DecoderModel
from ..weights.loader import load_tensors


def load_model(folder: str, dtype: str = "bfloat16", device: str | torch.device = "cuda:0",
               max_positions: Optional[int] = None, strict: bool = True) -> DecoderModel:
    """`strict=False`: tensors the model does not use are left alone with a warning instead of being an error."""
    dtype = canonical_dtype(dtype)
    config = load_config(folder)
    arch = lookup_architecture(config.architecture)
    model = arch.build(config, dtype=dtype, device=str(device), max_positions=max_positions)
    tensors = load_tensors(folder, model.tensor_specs(), strict=strict, ignorable=getattr(model, "ignorable_tensors", ()))
    model.bind(tensors, torch.device(device))
    return model
