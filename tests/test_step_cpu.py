"""The step function, the cache and the model assembly on the CPU, through the PyTorch
stand-in kernel set, against the plain implementation: whole prompts, token by token,
portions, and mixed batches with reused pages."""
import pytest
import torch

import replay_modes
from helpers import assert_close, make_runner, random_tokens
from plain_qwen2 import logits_of, read_folder
from tiny_configs import PAGE_SIZE, make_model_folder
from torch_kernels import TorchKernels

REL = 1e-4


def _runner(tmp_path, name, num_pages=64, **kw):
    folder = make_model_folder(tmp_path, name)
    runner = make_runner(folder, TorchKernels(), dtype="float32", device="cpu", page_size=PAGE_SIZE[name],
                         num_pages=num_pages, **kw)
    config, weights = read_folder(folder)
    return runner, config, weights


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompt(tmp_path, name):
    runner, config, weights = _runner(tmp_path, name)
    tokens = random_tokens(config["vocab_size"], 75, 1)
    assert_close(replay_modes.whole(runner, tokens), logits_of(config, weights, tokens), REL)
    assert runner.cache.used_pages() == 0


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_decode_one_by_one(tmp_path, name):
    runner, config, weights = _runner(tmp_path, name)
    tokens = random_tokens(config["vocab_size"], 90, 2)
    assert_close(replay_modes.last_32_one_by_one(runner, tokens), logits_of(config, weights, tokens)[-33:], REL)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_portions(tmp_path, name):
    runner, config, weights = _runner(tmp_path, name)
    tokens = random_tokens(config["vocab_size"], 101, 3)
    got = replay_modes.portions(runner, tokens, [2, 17, 3, 31, 2, 16, 8, 22])
    assert_close(got, logits_of(config, weights, tokens), REL)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_with_page_reuse(tmp_path, name):
    page = PAGE_SIZE[name]
    runner, config, weights = _runner(tmp_path, name, num_pages=replay_modes.mixed_pool_tokens() // page)
    seqs = {k: random_tokens(config["vocab_size"], n, 10 + i) for i, (k, n) in enumerate(replay_modes.MIXED_LENGTHS)}
    got = replay_modes.mixed(runner, seqs)
    for k, tokens in seqs.items():
        assert_close(got[k], logits_of(config, weights, tokens), REL, k)
