"""Configuration and registry: keys read from config.json, defaults, refusals."""
import json
import os

import pytest

import kvcache_b200  # noqa: F401  (registers the architecture)
from kvcache_b200.config import (ConfigError, EngineOptions, Qwen2Config, config_from_dict, load_config,
                                 lookup_architecture, register_architecture, registered_architectures,
                                 unregister_architecture)
from tiny_configs import CONFIGS, TINY_A, TINY_B, TINY_C


def test_keys_are_read_and_written_back():
    for data in CONFIGS.values():
        cfg = config_from_dict(data)
        assert isinstance(cfg, Qwen2Config)
        again = config_from_dict(cfg.to_dict())
        assert again == cfg
    a, b = config_from_dict(TINY_A), config_from_dict(TINY_B)
    assert (a.hidden_size, a.num_hidden_layers, a.num_attention_heads, a.num_key_value_heads) == (64, 2, 4, 2)
    assert a.head_dim == 16 and not a.explicit_head_dim          # derived: hidden / heads
    assert b.head_dim == 32 and b.explicit_head_dim
    assert a.eos_token_ids == (255,) and b.eos_token_ids == (382, 383)
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    assert (a.rms_norm_eps, b.rms_norm_eps, a.rope_theta, b.rope_theta) == (1e-6, 1e-5, 10000.0, 1000000.0)


def test_head_dim_may_differ_from_hidden_over_heads():
    c = config_from_dict(TINY_C)
    assert c.head_dim == 48 and c.q_size == 288 and c.kv_size == 96 and c.hidden_size == 120


def test_window_layers():
    c = config_from_dict(TINY_C)
    assert [c.layer_window(i) for i in range(4)] == [None, 40, 40, 40]
    assert all(config_from_dict(TINY_A).layer_window(i) is None for i in range(2))
    off = dict(TINY_C, use_sliding_window=False)
    assert all(config_from_dict(off).layer_window(i) is None for i in range(4))


def test_defaults():
    data = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "tie_word_embeddings", "eos_token_id",
                                                         "hidden_act", "max_window_layers")}
    c = config_from_dict(data)
    assert c.num_key_value_heads == c.num_attention_heads
    assert c.tie_word_embeddings is False and c.eos_token_ids == () and c.hidden_act == "silu"


def test_all_problems_are_reported_together():
    bad = dict(TINY_A)
    del bad["hidden_size"]
    bad["rms_norm_eps"] = "small"
    bad["num_key_value_heads"] = 3
    with pytest.raises(ConfigError) as err:
        config_from_dict(bad)
    text = str(err.value)
    assert "hidden_size" in text and "rms_norm_eps" in text and "multiple" in text


@pytest.mark.parametrize("change,word", [
    ({"hidden_act": "gelu"}, "hidden_act"), ({"rope_scaling": {"type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"head_dim": 15}, "even"), ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"), ({"hidden_size": 66, "head_dim": None}, "head_dim"),
])
def test_refusals(change, word):
    with pytest.raises(ConfigError, match=word):
        config_from_dict(dict(TINY_A, **change))


def test_unknown_architecture_and_registry():
    with pytest.raises(ConfigError, match="unknown architecture"):
        config_from_dict(dict(TINY_A, architectures=["SomethingElse"]))
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in TINY_A.items() if k != "architectures"})
    assert "Qwen2ForCausalLM" in registered_architectures()
    with pytest.raises(ValueError, match="already registered"):
        register_architecture("Qwen2ForCausalLM", Qwen2Config, lambda *a, **k: None)
    register_architecture("ToyForTests", Qwen2Config, lambda *a, **k: "built")
    try:
        assert lookup_architecture("ToyForTests").build() == "built"
    finally:
        unregister_architecture("ToyForTests")


def test_load_config_from_folder(tmp_path):
    with open(os.path.join(tmp_path, "config.json"), "w") as fh:
        json.dump(TINY_B, fh)
    assert load_config(str(tmp_path)).vocab_size == 384
    with pytest.raises(ConfigError, match="no such file"):
        load_config(os.path.join(tmp_path, "nowhere"))
    with open(os.path.join(tmp_path, "config.json"), "w") as fh:
        fh.write("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(str(tmp_path))


def test_engine_options():
    assert EngineOptions(dtype="bf16").dtype == "bfloat16" and EngineOptions(dtype="fp32").dtype == "float32"
    with pytest.raises(ValueError):
        EngineOptions(dtype="float16")
    with pytest.raises(ValueError):
        EngineOptions(page_size=12)
    with pytest.raises(ValueError):
        EngineOptions(admission="never")
