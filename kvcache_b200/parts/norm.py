"""RMSNorm with the residual add folded in (reference: src/qwen_kernels.cu:26-43 after :55-61)."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..weights.loader import TensorSpec
from .base import LayerContext, Norm


class RMSNorm(Norm):
    """y = v * rsqrt(mean(v^2) + eps) * weight, v = h + delta, in float32; the weight stays float32."""

    def __init__(self, width: int, eps: float, weight_name: str):
        self.width = width
        self.eps = float(eps)
        self.weight_name = weight_name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.weight_name: TensorSpec((self.width,))}

    def init_kinds(self) -> Dict[str, str]:
        return {self.weight_name: "ones_plus_normal"}

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        self.weight = tensors[self.weight_name].to(torch.float32).to(device).contiguous()

    def weight_bytes(self) -> int:
        return self.width * 4

    def add_norm(self, h, delta, out, ctx: LayerContext, rows=None) -> None:
        ctx.kernels.add_rmsnorm(h, delta, self.weight, self.eps, out, rows)

    def fold_params(self):
        return self.weight, self.eps
