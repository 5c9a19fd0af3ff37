"""Grouped-query attention over the paged cache: the mixer of this architecture.

Reference: the attention part of the layer loop, apps/qwen_serve.cu:102-110
(q/k/v projections with bias, rotation of q and k, write into the pool, causal
paged attention with scale 1/sqrt(D), output projection without bias).
"""
from __future__ import annotations

import math
from typing import Dict, Mapping, Optional

import torch

from ..weights.loader import TensorSpec
from .base import TORCH_DTYPES, LayerContext, Mixer, PagedKVSpec, PositionEncoding


class GQAAttention(Mixer):
    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int, *, qkv_bias: bool,
                 out_bias: bool, position: Optional[PositionEncoding], window: Optional[int], prefix: str,
                 dtype: str, scale: Optional[float] = None):
        if num_heads % num_kv_heads != 0:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if out_bias:
            raise ValueError("an output-projection bias is not supported")
        self.hidden, self.num_heads, self.num_kv_heads, self.head_dim = hidden, num_heads, num_kv_heads, head_dim
        self.qkv_bias = qkv_bias
        self.position = position
        self.window = window
        self.prefix = prefix
        self.dtype = TORCH_DTYPES[dtype]
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.q_size = num_heads * head_dim
        self.kv_size = num_kv_heads * head_dim
        self.w_qkv: Optional[torch.Tensor] = None
        self.b_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        p = self.prefix
        specs = {
            f"{p}q_proj.weight": TensorSpec((self.q_size, self.hidden)),
            f"{p}k_proj.weight": TensorSpec((self.kv_size, self.hidden)),
            f"{p}v_proj.weight": TensorSpec((self.kv_size, self.hidden)),
            f"{p}o_proj.weight": TensorSpec((self.hidden, self.q_size)),
        }
        if self.qkv_bias:
            specs[f"{p}q_proj.bias"] = TensorSpec((self.q_size,))
            specs[f"{p}k_proj.bias"] = TensorSpec((self.kv_size,))
            specs[f"{p}v_proj.bias"] = TensorSpec((self.kv_size,))
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        p = self.prefix
        # One projection for q, k and v: rows [q heads | k heads | v heads].
        self.w_qkv = torch.cat([tensors[f"{p}{n}_proj.weight"] for n in "qkv"], dim=0).to(self.dtype).to(device).contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors[f"{p}{n}_proj.bias"] for n in "qkv"], dim=0).to(torch.float32).to(device).contiguous()
        self.w_o = tensors[f"{p}o_proj.weight"].to(self.dtype).to(device).contiguous()
        # The folded projection of decode steps rotates inside the product and wants a second copy of the q/k/v weight
        # with each head's rows reordered (made when first asked for): possible in bfloat16, with whole-head rotation (or
        # none) and heads in steps of 16.
        self.w_qkv_paired = self.b_qkv_paired = None
        self._can_pair = self.dtype == torch.bfloat16 and self.head_dim % 16 == 0 and device.type == "cuda"

    def _pair_rows(self, kernels) -> bool:
        """Makes the row-paired copy of the q/k/v weight and bias if the kernel set can use one."""
        rotation = self.position.rotation() if self.position is not None else None
        whole = rotation is None or rotation.cos.shape[1] * 2 == self.head_dim
        if self.w_qkv_paired is None and self._can_pair and whole and hasattr(kernels, "pair_rotation_rows"):
            order = kernels.pair_rotation_rows(self.num_heads + 2 * self.num_kv_heads, self.head_dim).to(self.w_qkv.device)
            self.w_qkv_paired = self.w_qkv.index_select(0, order).contiguous()
            if self.b_qkv is not None:
                self.b_qkv_paired = self.b_qkv.index_select(0, order).contiguous()
        return self.w_qkv_paired is not None

    def weight_bytes(self) -> int:
        n = self.w_qkv.numel() * self.w_qkv.element_size() + self.w_o.numel() * self.w_o.element_size()
        return n + (self.b_qkv.numel() * 4 if self.b_qkv is not None else 0)

    def cache_spec(self) -> PagedKVSpec:
        return PagedKVSpec(self.num_kv_heads, self.head_dim, self.window)

    def step_planners(self, kernels):
        planner = getattr(kernels, "paged_attention_planner", None)
        return () if planner is None else (planner(),)

    def supports_fold(self, norm, kernels, num_rows: int) -> bool:
        can = getattr(kernels, "can_fold", None)
        return (can is not None and norm.fold_params() is not None
                and can(self.dtype, num_rows, self.hidden, self.q_size + 2 * self.kv_size)
                and can(self.dtype, num_rows, self.q_size, self.hidden) and self._pair_rows(kernels))

    def forward_folded(self, h: torch.Tensor, h16: torch.Tensor, norm, ctx: LayerContext) -> None:
        T = h.shape[0]
        k, ws = ctx.kernels, ctx.workspace
        weight, eps = norm.fold_params()
        rotation = self.position.rotation() if self.position is not None else None
        cos, sin = (rotation.cos, rotation.sin) if rotation else (None, None)
        q = ws.buffer("attn.q", (T, self.q_size), self.dtype)
        k.norm_qkv_rope_append(h16, self.w_qkv_paired, self.b_qkv_paired, weight, eps, cos, sin, ctx.batch, ctx.kv, q,
                               self.num_heads)
        attn = ws.buffer("attn.out", (T, self.q_size), self.dtype)
        k.paged_attention(q, ctx.batch, ctx.kv, attn, self.num_heads, self.scale, ws)
        k.linear_into_residual(attn, self.w_o, h, h16)


    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        T = x.shape[0]
        k, ws = ctx.kernels, ctx.workspace
        qkv = ws.buffer("attn.qkv", (T, self.q_size + 2 * self.kv_size), self.dtype)
        k.linear(x, self.w_qkv, qkv)
        rotation = self.position.rotation() if self.position is not None else None
        cos, sin = (rotation.cos, rotation.sin) if rotation else (None, None)
        attn = ws.buffer("attn.out", (T, self.q_size), self.dtype)
        # A kernel set may do bias, rotation, append and attention in one launch where it has a kernel for that.
        fused = getattr(k, "rope_append_attention", None)
        if fused is None or not fused(qkv, self.b_qkv, cos, sin, ctx.batch, ctx.kv, attn, self.num_heads, self.scale, ws):
            q = ws.buffer("attn.q", (T, self.q_size), self.dtype)
            k.qkv_rope_append(qkv, self.b_qkv, cos, sin, ctx.batch, ctx.kv, q, self.num_heads)
            k.paged_attention(q, ctx.batch, ctx.kv, attn, self.num_heads, self.scale, ws)
        delta = ws.buffer("attn.delta", (T, self.hidden), self.dtype)
        k.linear(attn, self.w_o, delta)
        return delta
