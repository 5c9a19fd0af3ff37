"""The arrangement of parts in one layer: pre-norm residual block
(reference order: apps/qwen_serve.cu:101-116)."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..weights.loader import TensorSpec
from .base import TORCH_DTYPES, Block, FeedForward, LayerContext, Mixer, Norm


class PreNormBlock(Block):
    """h += mixer(norm1(h)); h += ffn(norm2(h)).

    Each add is folded into the norm that follows it, so the block takes the
    previous layer's delta as `pending` and hands its own feed-forward delta on.
    """

    def __init__(self, width: int, norm1: Norm, mixer: Mixer, norm2: Norm, ffn: FeedForward, dtype: str):
        self.width = width
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self.dtype = TORCH_DTYPES[dtype]

    def _parts(self):
        return (self.norm1, self.mixer, self.norm2, self.ffn)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for part in self._parts():
            out.update(part.tensor_specs())
        return out

    def init_kinds(self) -> Dict[str, str]:
        out: Dict[str, str] = {}
        for part in self._parts():
            out.update(part.init_kinds())
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        for part in self._parts():
            part.bind(tensors, device)

    def weight_bytes(self) -> int:
        return sum(part.weight_bytes() for part in self._parts())

    def supports_fold(self, kernels, num_rows: int) -> bool:
        return (self.mixer.supports_fold(self.norm1, kernels, num_rows)
                and self.ffn.supports_fold(self.norm2, kernels, num_rows))

    def forward_folded(self, h: torch.Tensor, h16: torch.Tensor, ctx: LayerContext) -> None:
        self.mixer.forward_folded(h, h16, self.norm1, ctx)
        self.ffn.forward_folded(h, h16, self.norm2, ctx)

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], ctx: LayerContext) -> Optional[torch.Tensor]:
        T = h.shape[0]
        x = ctx.workspace.buffer("block.normed", (T, self.width), self.dtype)
        self.norm1.add_norm(h, pending, x, ctx)
        delta = self.mixer.forward(x, ctx)
        self.norm2.add_norm(h, delta, x, ctx)
        return self.ffn.forward(x, ctx)
