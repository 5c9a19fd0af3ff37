from .attention import GQAAttention
from .base import (Block, FeedForward, LayerContext, Mixer, Norm, PagedKVSpec, PagedKVView, Part,
                   PositionEncoding, Rotation, StateSpec, StepBatch, StepPlan, StepPlanner, TORCH_DTYPES)
from .block import PreNormBlock
from .feedforward import GatedMLP
from .model import CacheEntry, DecoderModel, LayerCall
from .norm import RMSNorm
from .position import NoPositionEncoding, RotaryHalf

__all__ = ["GQAAttention", "Block", "FeedForward", "LayerContext", "Mixer", "Norm", "PagedKVSpec",
           "PagedKVView", "Part", "PositionEncoding", "Rotation", "StateSpec", "StepBatch", "StepPlan", "StepPlanner", "TORCH_DTYPES",
           "PreNormBlock", "GatedMLP", "CacheEntry", "DecoderModel", "LayerCall", "RMSNorm",
           "NoPositionEncoding", "RotaryHalf"]
