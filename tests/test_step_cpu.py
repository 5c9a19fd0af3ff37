"""The step function, the cache and the model assembly on the CPU, through the PyTorch
stand-in kernel set, against the plain implementation: whole prompts, token by token,
portions, and mixed batches with reused pages."""
import pytest
import torch

from helpers import make_runner, random_tokens
from plain_qwen2 import logits_of, read_folder
from tiny_configs import CONFIGS, PAGE_SIZE, make_model_folder
from torch_kernels import TorchKernels

from kvcache_b200.engine.runner import StepEntry

TOL = 2e-4


def _runner(tmp_path, name, num_pages=64, **kw):
    folder = make_model_folder(tmp_path, name)
    runner = make_runner(folder, TorchKernels(), dtype="float32", device="cpu", page_size=PAGE_SIZE[name],
                         num_pages=num_pages, **kw)
    config, weights = read_folder(folder)
    return runner, config, weights


def _close(got, want):
    want = want.to(torch.float32)
    err = (got - want).abs().max().item()
    assert err <= TOL * max(1.0, want.abs().max().item()), f"max abs error {err}"


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompt(tmp_path, name):
    runner, config, weights = _runner(tmp_path, name)
    tokens = random_tokens(config["vocab_size"], 75, 1)
    slot = runner.cache.admit()
    got = runner.step([StepEntry(slot, tokens, list(range(len(tokens))))]).clone()
    _close(got, logits_of(config, weights, tokens))
    runner.cache.release(slot)
    assert runner.cache.used_pages() == 0


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_decode_one_by_one(tmp_path, name):
    runner, config, weights = _runner(tmp_path, name)
    tokens = random_tokens(config["vocab_size"], 90, 2)
    want = logits_of(config, weights, tokens)
    slot = runner.cache.admit()
    head = len(tokens) - 32
    got = [runner.step([StepEntry(slot, tokens[:head], [head - 1])]).clone()]
    for i in range(head, len(tokens)):
        got.append(runner.step([StepEntry(slot, tokens[i:i + 1], [0])]).clone())
    _close(torch.cat(got), want[head - 1:])


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_portions(tmp_path, name):
    runner, config, weights = _runner(tmp_path, name)
    tokens = random_tokens(config["vocab_size"], 101, 3)
    want = logits_of(config, weights, tokens)
    slot = runner.cache.admit()
    got, at = [], 0
    for size in [2, 17, 3, 31, 2, 16, 8, 22]:
        piece = tokens[at:at + size]
        got.append(runner.step([StepEntry(slot, piece, list(range(len(piece))))]).clone())
        at += len(piece)
    assert at == len(tokens)
    _close(torch.cat(got), want)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_with_page_reuse(tmp_path, name):
    page = PAGE_SIZE[name]
    runner, config, weights = _runner(tmp_path, name, num_pages=(64 * 3 + 48) // page)
    V = config["vocab_size"]
    seqs = {k: random_tokens(V, n, 10 + i) for i, (k, n) in enumerate([("a", 60), ("b", 37), ("c", 64), ("d", 45), ("e", 50)])}
    want = {k: logits_of(config, weights, v) for k, v in seqs.items()}
    slots, done = {}, {k: 0 for k in seqs}
    got = {k: [] for k in seqs}

    def run(parts):
        entries = []
        for k, n in parts:
            if k not in slots:
                slots[k] = runner.cache.admit()
            entries.append(StepEntry(slots[k], seqs[k][done[k]:done[k] + n], list(range(n))))
        out = runner.step(entries).clone()
        at = 0
        for k, n in parts:
            got[k].append(out[at:at + n])
            at += n
            done[k] += n

    def end(k):
        runner.cache.release(slots.pop(k))

    run([("a", 30), ("b", 5)])
    run([("a", 1), ("b", 20), ("c", 33)])
    run([("a", 1), ("b", 12), ("c", 2)])
    run([("a", 28), ("c", 29)])
    end("a"); end("b")
    run([("d", 45), ("e", 7)])      # d and e take the pages a and b gave back
    run([("e", 2)])
    end("c")
    run([("e", 41)])
    for k in list(slots):
        end(k)
    assert runner.cache.used_pages() == 0
    for k in seqs:
        assert done[k] == len(seqs[k]), k
        _close(torch.cat(got[k]), want[k])
