"""Dense gated feed-forward (reference: apps/qwen_serve.cu:112-116, src/qwen_kernels.cu:102-105)."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..weights.loader import TensorSpec
from .base import TORCH_DTYPES, FeedForward, LayerContext


class GatedMLP(FeedForward):
    """delta = (act(x Wg^T) * (x Wu^T)) Wd^T with act = silu; no biases."""

    def __init__(self, hidden: int, intermediate: int, *, activation: str, prefix: str, dtype: str):
        if activation != "silu":
            raise ValueError(f"activation '{activation}' is not supported by the gated feed-forward kernel")
        self.hidden, self.intermediate = hidden, intermediate
        self.prefix = prefix
        self.dtype = TORCH_DTYPES[dtype]
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None
        self.interleaved = False

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        p = self.prefix
        return {
            f"{p}gate_proj.weight": TensorSpec((self.intermediate, self.hidden)),
            f"{p}up_proj.weight": TensorSpec((self.intermediate, self.hidden)),
            f"{p}down_proj.weight": TensorSpec((self.hidden, self.intermediate)),
        }

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        p = self.prefix
        gate, up = tensors[f"{p}gate_proj.weight"], tensors[f"{p}up_proj.weight"]
        # One projection for gate and up.  When the width allows, rows are interleaved in eights (gate rows
        # 8 b .. 8 b + 7, then the up rows of the same indices) so that a kernel's thread holds both values
        # of an index and can write the activation without a second pass.
        self.interleaved = self.intermediate % 8 == 0
        if self.interleaved:
            both = torch.stack([gate.view(-1, 8, self.hidden), up.view(-1, 8, self.hidden)], dim=1).reshape(-1, self.hidden)
        else:
            both = torch.cat([gate, up], dim=0)
        self.w_gate_up = both.to(self.dtype).to(device).contiguous()
        self.w_down = tensors[f"{p}down_proj.weight"].to(self.dtype).to(device).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def supports_fold(self, norm, kernels, num_rows: int) -> bool:
        can = getattr(kernels, "can_fold", None)
        return (can is not None and self.interleaved and norm.fold_params() is not None
                and can(self.dtype, num_rows, self.hidden, 2 * self.intermediate)
                and can(self.dtype, num_rows, self.intermediate, self.hidden))

    def forward_folded(self, h: torch.Tensor, h16: torch.Tensor, norm, ctx: LayerContext) -> None:
        T = h.shape[0]
        k, ws = ctx.kernels, ctx.workspace
        weight, eps = norm.fold_params()
        act = ws.buffer("ffn.act", (T, self.intermediate), self.dtype)
        k.norm_gate_up_act(h16, self.w_gate_up, weight, eps, act)
        k.linear_into_residual(act, self.w_down, h, h16)


    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        T = x.shape[0]
        k, ws = ctx.kernels, ctx.workspace
        act = ws.buffer("ffn.act", (T, self.intermediate), self.dtype)
        k.gate_up_act(x, self.w_gate_up, act, ws, self.interleaved)
        delta = ws.buffer("ffn.delta", (T, self.hidden), self.dtype)
        k.linear(act, self.w_down, delta)
        return delta
