"""The tiny configurations the tests use: they differ in every size and option."""
from __future__ import annotations

import os

import torch

TINY_A = {  # 2 layers, tied head, no window, page 16
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2,
    "intermediate_size": 128, "vocab_size": 256, "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
    "tie_word_embeddings": True, "max_position_embeddings": 512, "hidden_act": "silu",
    "use_sliding_window": False, "sliding_window": None, "max_window_layers": 2, "eos_token_id": 255,
}
TINY_B = {  # 3 layers, one kv head (group of 3), untied head, explicit head_dim, page 8
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "hidden_size": 96, "num_hidden_layers": 3, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 320, "vocab_size": 384, "rms_norm_eps": 1e-5, "rope_theta": 1000000.0,
    "tie_word_embeddings": False, "max_position_embeddings": 1024, "hidden_act": "silu",
    "use_sliding_window": False, "sliding_window": None, "max_window_layers": 3, "eos_token_id": [382, 383],
}
TINY_C = {  # sizes that are no power of two anywhere; windowed upper layers; head_dim 48 != hidden / heads
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "hidden_size": 120, "num_hidden_layers": 4, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 48, "intermediate_size": 200, "vocab_size": 331, "rms_norm_eps": 3e-6, "rope_theta": 50000.0,
    "tie_word_embeddings": False, "max_position_embeddings": 768, "hidden_act": "silu",
    "use_sliding_window": True, "sliding_window": 40, "max_window_layers": 1, "initializer_range": 0.05,
}
TINY_D = {  # head size 64, the size of the benchmarked model: the TMA decode and tensor-memory prefill kernels; group of 7
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "hidden_size": 112, "num_hidden_layers": 2, "num_attention_heads": 7, "num_key_value_heads": 1,
    "head_dim": 64, "intermediate_size": 136, "vocab_size": 270, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "tie_word_embeddings": True, "max_position_embeddings": 2048, "hidden_act": "silu",
    "use_sliding_window": True, "sliding_window": 300, "max_window_layers": 1,
}
PAGE_SIZE = {"A": 16, "B": 8, "C": 16, "D": 32}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}


def make_model_folder(tmp_path, name: str, seed: int = 0, dtype=torch.float32) -> str:
    """Writes a random-weights folder for tiny configuration `name` under tmp_path."""
    import kvcache_b200  # registers the architecture
    from kvcache_b200.config import config_from_dict
    from kvcache_b200.weights import write_random_model
    folder = os.path.join(str(tmp_path), f"tiny_{name}_{seed}")
    write_random_model(folder, config_from_dict(CONFIGS[name]), seed, dtype)
    return folder
