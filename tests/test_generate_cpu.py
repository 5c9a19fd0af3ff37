"""Generation through the Python entry point on the CPU stand-in kernels: greedy tokens equal
the plain implementation's, whatever the batching; temperature runs repeat from their seed."""
import pytest
import torch

from helpers import random_tokens
from plain_qwen2 import greedy_generate, read_folder
from tiny_configs import PAGE_SIZE, make_model_folder
from torch_kernels import TorchKernels

from kvcache_b200 import LLM, SamplingParams


def _llm(folder, name, **kw):
    fields = dict(dtype="float32", device="cpu", page_size=PAGE_SIZE[name], num_pages=64, max_running=4,
                  max_tokens_per_step=64, chunk_size=16, use_graphs=False)
    fields.update(kw)
    return LLM(folder, kernels=TorchKernels(), **fields)


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_matches_plain(tmp_path, name):
    folder = make_model_folder(tmp_path, name)
    config, weights = read_folder(folder)
    lengths = [5, 17, 33] if name == "A" else [1, 9, 24, 40, 63]
    prompts = [random_tokens(config["vocab_size"], n, 40 + n) for n in lengths]
    llm = _llm(folder, name)
    got = llm.generate(prompts, SamplingParams(max_new_tokens=8, ignore_eos=True))
    for prompt, out in zip(prompts, got):
        assert out == greedy_generate(config, weights, prompt, 8)
    assert llm.core.cache.used_pages() == 0
    stats = llm.last_stats
    assert stats.finished == len(prompts) and stats.generated == 8 * len(prompts)


def test_temperature_is_reproducible_and_batch_invariant(tmp_path):
    folder = make_model_folder(tmp_path, "B")
    config, _ = read_folder(folder)
    prompts = [random_tokens(config["vocab_size"], n, 50 + n) for n in (1, 9, 24, 40, 63)]
    params = [SamplingParams(max_new_tokens=12, temperature=0.7, seed=100 + i, ignore_eos=True) for i in range(5)]
    first = _llm(folder, "B").generate(prompts, params)
    again = _llm(folder, "B", max_running=2, chunk_size=7, max_tokens_per_step=20).generate(prompts, params)
    assert first == again
    other = _llm(folder, "B").generate(prompts, [SamplingParams(max_new_tokens=12, temperature=0.7, seed=7 + i,
                                                               ignore_eos=True) for i in range(5)])
    assert first != other


def test_eos_ends_a_request_and_is_kept(tmp_path):
    folder = make_model_folder(tmp_path, "A")
    config, weights = read_folder(folder)
    prompt = random_tokens(config["vocab_size"], 12, 60)
    free_run = greedy_generate(config, weights, prompt, 10)
    stop = free_run[3]
    got = _llm(folder, "A").generate([prompt], SamplingParams(max_new_tokens=10, eos_token_ids=(stop,)))[0]
    assert got == free_run[:free_run.index(stop) + 1]
