"""The engine on the GPU with its CUDA kernels, in float32 and in bfloat16, against the plain
implementation: each request alone and whole; most of it in one step and the last 32 tokens
one by one; portions of changing size down to two tokens; mixed batches with reused pages;
long decoding; the first tokens of a sequence."""
import pytest
import torch

import replay_modes
from helpers import assert_close, make_runner, random_tokens
from plain_qwen2 import logits_of, read_folder
from tiny_configs import PAGE_SIZE, make_model_folder

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# Relative to the largest logit of the reference.  float32: summation order only.
# bfloat16: weights are exact in both (the folder is written in bfloat16); what differs is the
# rounding of activations to 8 bits of mantissa at every matrix product's input and output.
REL = {"float32": 1e-4, "bfloat16": 3e-2}
NAMES = ["A", "B", "C"]
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def kernels():
    from kvcache_b200.kernels.api import CudaKernels
    return CudaKernels(DEV)


def _runner(tmp_path, kernels, name, dtype, num_pages=64, **kw):
    folder = make_model_folder(tmp_path, name, dtype=torch.bfloat16)
    runner = make_runner(folder, kernels, dtype=dtype, device=DEV, page_size=PAGE_SIZE[name],
                         num_pages=num_pages, **kw)
    config, weights = read_folder(folder)
    return runner, config, weights


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompt(tmp_path, kernels, name, dtype):
    runner, config, weights = _runner(tmp_path, kernels, name, dtype)
    for n, seed in [(75, 1), (1, 2), (16, 3), (129, 4)]:
        tokens = random_tokens(config["vocab_size"], n, seed)
        assert_close(replay_modes.whole(runner, tokens), logits_of(config, weights, tokens), REL[dtype], f"n={n}")
    kernels.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_one_by_one(tmp_path, kernels, name, dtype):
    runner, config, weights = _runner(tmp_path, kernels, name, dtype)
    tokens = random_tokens(config["vocab_size"], 90, 5)
    assert_close(replay_modes.last_32_one_by_one(runner, tokens), logits_of(config, weights, tokens)[-33:], REL[dtype])
    kernels.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions(tmp_path, kernels, name, dtype):
    runner, config, weights = _runner(tmp_path, kernels, name, dtype)
    tokens = random_tokens(config["vocab_size"], 101, 6)
    want = logits_of(config, weights, tokens)
    for sizes in ([2, 17, 3, 31, 2, 16, 8, 22], [50, 2, 2, 2, 45], [1] * 5 + [96]):
        assert_close(replay_modes.portions(runner, tokens, sizes), want, REL[dtype], str(sizes))
    kernels.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_with_page_reuse(tmp_path, kernels, name, dtype):
    page = PAGE_SIZE[name]
    runner, config, weights = _runner(tmp_path, kernels, name, dtype,
                                      num_pages=replay_modes.mixed_pool_tokens() // page)
    seqs = {k: random_tokens(config["vocab_size"], n, 10 + i) for i, (k, n) in enumerate(replay_modes.MIXED_LENGTHS)}
    got = replay_modes.mixed(runner, seqs)
    for k, tokens in seqs.items():
        assert_close(got[k], logits_of(config, weights, tokens), REL[dtype], k)
    kernels.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "C"])
def test_long_decoding(tmp_path, kernels, name, dtype):
    """300 tokens decoded one by one after a short prompt: every page edge and, for the
    windowed configuration, pages given back behind the window."""
    runner, config, weights = _runner(tmp_path, kernels, name, dtype, num_pages=48)
    tokens = random_tokens(config["vocab_size"], 310, 7)
    want = logits_of(config, weights, tokens)
    from kvcache_b200.engine.runner import StepEntry
    slot = runner.cache.admit()
    got = [runner.step([StepEntry(slot, tokens[:10], list(range(10)))]).clone()]
    for i in range(10, len(tokens)):
        got.append(runner.step([StepEntry(slot, tokens[i:i + 1], [0])]).clone())
    assert_close(torch.cat(got), want, REL[dtype])
    if config.get("use_sliding_window"):
        window_group = [g for g in runner.cache.groups if g.spec.window][0]
        assert len(window_group.pages.held_pages(slot)) <= (config["sliding_window"] + PAGE_SIZE[name]) // PAGE_SIZE[name] + 1
    kernels.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_composition_does_not_change_logits(tmp_path, kernels, dtype):
    """The same request alone and beside three others: equal beyond rounding."""
    runner, config, weights = _runner(tmp_path, kernels, "B", dtype)
    from kvcache_b200.engine.runner import StepEntry
    V = config["vocab_size"]
    a = random_tokens(V, 40, 20)
    alone = replay_modes.whole(runner, a)
    others = [random_tokens(V, n, 21 + n) for n in (3, 25, 9)]
    slots = [runner.cache.admit() for _ in range(4)]
    entries = [StepEntry(slots[1], others[0], []), StepEntry(slots[0], a, list(range(40))),
               StepEntry(slots[2], others[1], [0]), StepEntry(slots[3], others[2], [])]
    together = runner.step(entries).clone()[:40]
    assert_close(together, alone, 1e-5 if dtype == "float32" else 2e-2)
