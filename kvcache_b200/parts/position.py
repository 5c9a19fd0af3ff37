"""Position encodings.  The one this architecture uses rotates queries and keys
(rotate-half pairing; reference: src/qwen_kernels.cu:63-78, per-row positions :253-264)."""
from __future__ import annotations

from typing import Mapping, Optional

import numpy as np
import torch

from .base import PositionEncoding, Rotation


class RotaryHalf(PositionEncoding):
    """Pairs dimension t with t + rotary_dim/2; angle = pos * theta^(-2t / rotary_dim).

    The cos/sin tables for positions 0..max_positions-1 are made once on the
    host in double precision and rounded to float32, so the angle of a far
    position carries no accumulated float32 error.
    """

    def __init__(self, rotary_dim: int, theta: float, max_positions: int):
        if rotary_dim % 2 != 0 or rotary_dim < 2:
            raise ValueError(f"rotary_dim must be even and positive, got {rotary_dim}")
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        self._rotation: Optional[Rotation] = None

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        half = self.rotary_dim // 2
        inv_freq = self.theta ** (-(np.arange(half, dtype=np.float64) * 2.0) / self.rotary_dim)
        angles = np.arange(self.max_positions, dtype=np.float64)[:, None] * inv_freq[None, :]
        cos = torch.from_numpy(np.cos(angles).astype(np.float32)).to(device).contiguous()
        sin = torch.from_numpy(np.sin(angles).astype(np.float32)).to(device).contiguous()
        self._rotation = Rotation(cos=cos, sin=sin)

    def rotation(self) -> Optional[Rotation]:
        return self._rotation


class NoPositionEncoding(PositionEncoding):
    pass
