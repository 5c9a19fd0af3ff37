"""Configuration of the Qwen2 dense decoder, read from its own config.json keys.

The keys are those the reference copies out of the checkpoint
(tools/dump_weights.py:46-58) and hard-codes for Qwen2.5-0.5B
(apps/qwen_serve.cu:20-23: H, Hq, Hkv, D, IM, NL, VOCAB, EPS, THETA, EOS ids),
plus the window keys that the same config.json carries
(`use_sliding_window`, `sliding_window`, `max_window_layers`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .base import KeyReader, ModelConfig

QWEN2_ARCHITECTURE = "Qwen2ForCausalLM"


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    hidden_act: str
    use_sliding_window: bool
    sliding_window: Optional[int]
    max_window_layers: int
    eos_token_ids: Tuple[int, ...]
    initializer_range: float
    # True when config.json spelled head_dim out (it is written back only then).
    explicit_head_dim: bool = False

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str = "config.json") -> "Qwen2Config":
        r = KeyReader(data, where)
        hidden = r.integer("hidden_size", minimum=1)
        layers = r.integer("num_hidden_layers", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        kv_heads = r.integer("num_key_value_heads", default=heads, minimum=1)
        inter = r.integer("intermediate_size", minimum=1)
        vocab = r.integer("vocab_size", minimum=1)
        eps = r.number("rms_norm_eps", positive=True)
        theta = r.number("rope_theta", positive=True)
        tie = r.boolean("tie_word_embeddings", default=False)
        max_pos = r.integer("max_position_embeddings", minimum=1)
        act = r.string("hidden_act", default="silu")
        use_window = r.boolean("use_sliding_window", default=False)
        window = r.integer("sliding_window", default=None, minimum=1)
        max_window_layers = r.integer("max_window_layers", default=layers, minimum=0)
        eos = r.int_list("eos_token_id", default=())
        init_range = r.number("initializer_range", default=0.02, positive=True)
        explicit_head_dim = data.get("head_dim") is not None
        head_dim = r.integer("head_dim", default=None, minimum=1)

        if head_dim is None and hidden is not None and heads is not None:
            # tools/dump_weights.py:52 derives it the same way.
            if hidden % heads != 0:
                r.fail(f"hidden_size {hidden} is not a multiple of num_attention_heads {heads} and no head_dim is given")
            else:
                head_dim = hidden // heads
        if head_dim is not None and head_dim % 2 != 0:
            r.fail(f"head_dim {head_dim} must be even (rotate-half pairs dimension t with t + head_dim/2)")
        if heads is not None and kv_heads is not None and heads % kv_heads != 0:
            r.fail(f"num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        if act is not None and act != "silu":
            r.fail(f"hidden_act '{act}' is not supported (the gated feed-forward of this architecture uses 'silu')")
        if data.get("rope_scaling") not in (None, {}):
            r.fail("rope_scaling is not supported")
        if use_window and window is None:
            r.fail("use_sliding_window is true but sliding_window is not given")
        r.finish()
        return cls(
            architecture=QWEN2_ARCHITECTURE,
            hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
            num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=inter,
            vocab_size=vocab, rms_norm_eps=eps, rope_theta=theta, tie_word_embeddings=tie,
            max_position_embeddings=max_pos, hidden_act=act, use_sliding_window=use_window,
            sliding_window=window, max_window_layers=max_window_layers, eos_token_ids=eos,
            initializer_range=init_range, explicit_head_dim=explicit_head_dim,
        )

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen2",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
            "hidden_act": self.hidden_act,
            "use_sliding_window": self.use_sliding_window,
            "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers,
            "initializer_range": self.initializer_range,
        }
        if self.explicit_head_dim:
            out["head_dim"] = self.head_dim
        if len(self.eos_token_ids) == 1:
            out["eos_token_id"] = self.eos_token_ids[0]
        elif len(self.eos_token_ids) > 1:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out

    # ---- derived quantities -------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def layer_window(self, layer: int) -> Optional[int]:
        """Number of keys (its own included) a query of this layer sees, or None for all.

        The first `max_window_layers` layers attend to every key; the layers
        after them use the window when `use_sliding_window` is on.
        """
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None
