"""Qwen2 dense decoder put together from parts, layer by layer, from its configuration.

Layer sequence and tensor names as the reference runs them (apps/qwen_serve.cu:97-119):
embedding; per layer input_layernorm, q/k/v projections with bias, rotation,
attention, o_proj, post_attention_layernorm, gate/up/down; model.norm; lm_head
(the embedding table when tied).
"""
from __future__ import annotations

from typing import Optional

from ..config.qwen2 import QWEN2_ARCHITECTURE, Qwen2Config
from ..config.registry import register_architecture
from ..parts.attention import GQAAttention
from ..parts.block import PreNormBlock
from ..parts.feedforward import GatedMLP
from ..parts.model import DecoderModel, LayerCall
from ..parts.norm import RMSNorm
from ..parts.position import RotaryHalf


def build_qwen2(config: Qwen2Config, dtype: str = "bfloat16", device: str = "cuda:0",
                max_positions: Optional[int] = None) -> DecoderModel:
    c = config
    position = RotaryHalf(c.head_dim, c.rope_theta, max_positions or c.max_position_embeddings)
    blocks = []
    for i in range(c.num_hidden_layers):
        p = f"model.layers.{i}."
        blocks.append(PreNormBlock(
            c.hidden_size,
            RMSNorm(c.hidden_size, c.rms_norm_eps, p + "input_layernorm.weight"),
            GQAAttention(c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
                         qkv_bias=True, out_bias=False, position=position, window=c.layer_window(i),
                         prefix=p + "self_attn.", dtype=dtype),
            RMSNorm(c.hidden_size, c.rms_norm_eps, p + "post_attention_layernorm.weight"),
            GatedMLP(c.hidden_size, c.intermediate_size, activation=c.hidden_act, prefix=p + "mlp.", dtype=dtype),
            dtype))
    return DecoderModel(
        config=c, dtype=dtype, vocab_size=c.vocab_size, width=c.hidden_size,
        embed_name="model.embed_tokens.weight",
        head_name=None if c.tie_word_embeddings else "lm_head.weight",
        blocks=blocks, schedule=[LayerCall(i, i) for i in range(c.num_hidden_layers)],
        final_norm=RMSNorm(c.hidden_size, c.rms_norm_eps, "model.norm.weight"), position=position,
        # Checkpoints may carry the rotation's frequencies as a buffer, and the reference's exporter stores the embedding
        # a second time as lm_head.weight when the head is tied (tools/dump_weights.py:24-26): neither is used.
        ignorable_tensors=["*.rotary_emb.inv_freq"] + (["lm_head.weight"] if c.tie_word_embeddings else []))


register_architecture(QWEN2_ARCHITECTURE, Qwen2Config, build_qwen2, replace=True)
