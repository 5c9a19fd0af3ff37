"""The engine at the layer shapes of the family's larger members (hidden 1536 and 3584, head size 128, groups of 6
and 7 query heads, intermediate 8960 and 18944), two layers and a small vocabulary each, against the plain
implementation: whole, in portions, the last 32 tokens one by one, and mixed with reused pages."""
import os

import pytest
import torch

import replay_modes
from helpers import assert_close, make_runner, random_tokens
from plain_qwen2 import logits_of, read_folder

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REL = {"float32": 1e-4, "bfloat16": 3e-2}     # as for the tiny configurations
BASE = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
        "max_position_embeddings": 32768, "hidden_act": "silu", "use_sliding_window": False, "sliding_window": None,
        "num_hidden_layers": 2, "max_window_layers": 2, "vocab_size": 2003}
SHAPES = {
    "1.5B": dict(hidden_size=1536, num_attention_heads=12, num_key_value_heads=2, intermediate_size=8960,
                 tie_word_embeddings=True),
    "7B": dict(hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944,
               tie_word_embeddings=False),
}


@pytest.fixture(scope="module")
def kernels():
    from kvcache_b200.kernels.api import CudaKernels
    return CudaKernels(DEV)


@pytest.fixture(scope="module", params=list(SHAPES))
def family_model(request, tmp_path_factory):
    import kvcache_b200  # noqa: F401  (registers the architecture)
    from kvcache_b200.config import config_from_dict
    from kvcache_b200.weights import write_random_model
    folder = os.path.join(str(tmp_path_factory.mktemp("family")), request.param)
    write_random_model(folder, config_from_dict(dict(BASE, **SHAPES[request.param])), seed=1, dtype=torch.bfloat16)
    config, weights = read_folder(folder)
    tokens = random_tokens(config["vocab_size"], 700, 5)
    mixed = {k: random_tokens(config["vocab_size"], n, 10 + i) for i, (k, n) in enumerate(replay_modes.MIXED_LENGTHS)}
    want = {"tokens": logits_of(config, weights, tokens), **{k: logits_of(config, weights, t) for k, t in mixed.items()}}
    return folder, tokens, mixed, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_family_layer_shapes(family_model, kernels, dtype):
    folder, tokens, mixed, want = family_model
    runner = make_runner(folder, kernels, dtype=dtype, device=DEV, page_size=16, num_pages=64,
                         max_tokens_per_step=1024, max_tokens_per_request=1024)
    assert_close(replay_modes.whole(runner, tokens), want["tokens"], REL[dtype], "whole")
    assert_close(replay_modes.portions(runner, tokens, [450, 2, 130, 17, 101]), want["tokens"], REL[dtype], "portions")
    assert_close(replay_modes.last_32_one_by_one(runner, tokens), want["tokens"][-33:], REL[dtype], "last 32")
    assert runner.cache.used_pages() == 0
    del runner
    torch.cuda.empty_cache()
    small = make_runner(folder, kernels, dtype=dtype, device=DEV, page_size=16,
                        num_pages=replay_modes.mixed_pool_tokens() // 16)
    got = replay_modes.mixed(small, mixed)
    for k in mixed:
        assert_close(got[k], want[k], REL[dtype], k)
    kernels.check_errors()
