"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a
configuration and a seed.

The reference has no such mode (it needs a downloaded checkpoint,
tools/dump_weights.py:19).  Values: matrices and biases N(0, initializer_range),
norm weights 1 + N(0, initializer_range); every tensor draws from a generator
keyed by the seed and its own name, so that a tensor's values do not depend on
which other tensors exist.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Mapping, Optional

import torch

from ..config.base import ModelConfig
from .loader import FLOAT, TensorSpec
from .safetensors_io import write_safetensors


def _generator(seed: int, name: str) -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(digest[:8], "little") & ((1 << 63) - 1))
    return g


def random_tensors(specs: Mapping[str, TensorSpec], seed: int, std: float,
                   dtype: torch.dtype = torch.bfloat16,
                   init_kinds: Optional[Mapping[str, str]] = None) -> Dict[str, torch.Tensor]:
    """`init_kinds[name]` is "normal" (default), "ones_plus_normal" (norm weights) or "skip"."""
    out: Dict[str, torch.Tensor] = {}
    for name, spec in specs.items():
        kind = (init_kinds or {}).get(name, "normal")
        if kind == "skip":
            continue
        if spec.kind != FLOAT:
            raise ValueError(f"no random initialisation for integer tensor '{name}'")
        values = torch.randn(spec.shape, generator=_generator(seed, name), dtype=torch.float32) * std
        if kind == "ones_plus_normal":
            values = values + 1.0
        out[name] = values.to(dtype)
    return out


def write_random_model(folder: str, config: ModelConfig, seed: int,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Creates `folder` with config.json and model.safetensors for `config`; returns the folder."""
    from ..config.registry import lookup_architecture
    arch = lookup_architecture(config.architecture)
    model = arch.build(config, dtype="float32", device="meta")
    specs = model.tensor_specs()
    kinds = model.init_kinds()
    std = float(getattr(config, "initializer_range", 0.02))
    tensors = random_tensors(specs, seed, std, dtype, kinds)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(config.to_dict(), fh, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return folder
