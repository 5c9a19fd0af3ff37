"""Generation through the Python entry point and the command lines on the GPU."""
import os
import subprocess
import sys

import pytest
import torch

from helpers import random_tokens
from plain_qwen2 import greedy_generate, logits_of, read_folder
from tiny_configs import PAGE_SIZE, make_model_folder

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _llm(folder, name, dtype, **kw):
    from kvcache_b200 import LLM
    fields = dict(dtype=dtype, page_size=PAGE_SIZE[name], num_pages=64, max_running=4, max_tokens_per_step=64,
                  chunk_size=16, use_graphs=True)
    fields.update(kw)
    llm = LLM(folder, **fields)
    llm.core.runner.graph_after_sightings = 2      # so that these short runs replay portions, alone and beside decoded tokens
    return llm


def _greedy_follows_plain(config, weights, prompt, out, rel):
    """Every generated token against the plain implementation's logits for the sequence so far.  `rel` is the bound on
    the engine's logit error, as a fraction of the largest logit (the tolerance of the logit tests).  Where the plain
    first choice leads the second by more than twice that bound the engine must have made the same choice; elsewhere
    its choice must at least lie within twice the bound of the best.  Returns how many places were clear."""
    logits = logits_of(config, weights, list(prompt) + list(out[:-1]))[len(prompt) - 1:]
    clear = 0
    for i, t in enumerate(out):
        row = logits[i]
        bound = 2 * rel * row.abs().max().item()
        top = torch.topk(row, 2)
        if (top.values[0] - top.values[1]).item() > bound:
            clear += 1
            assert t == int(top.indices[0]), (i, t, int(top.indices[0]))
        else:
            assert row[t].item() >= top.values[0].item() - bound, (i, t, int(top.indices[0]))
    return clear


@pytest.mark.parametrize("use_graphs", [False, True])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_float32_equals_plain(tmp_path, name, use_graphs):
    from kvcache_b200 import SamplingParams
    folder = make_model_folder(tmp_path, name, dtype=torch.bfloat16)
    config, weights = read_folder(folder)
    lengths = [5, 17, 33] if name == "A" else [1, 9, 24, 40, 63]
    prompts = [random_tokens(config["vocab_size"], n, 70 + n) for n in lengths]
    llm = _llm(folder, name, "float32", use_graphs=use_graphs)
    got = llm.generate(prompts, SamplingParams(max_new_tokens=8, ignore_eos=True))
    for prompt, out in zip(prompts, got):
        assert out == greedy_generate(config, weights, prompt, 8)
    assert llm.core.cache.used_pages() == 0
    if use_graphs:
        assert llm.core.runner.graph_replays > 0


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_bfloat16_follows_plain(tmp_path, name):
    from kvcache_b200 import SamplingParams
    folder = make_model_folder(tmp_path, name, dtype=torch.bfloat16)
    config, weights = read_folder(folder)
    prompts = [random_tokens(config["vocab_size"], n, 80 + n) for n in (3, 30, 50)]
    got = _llm(folder, name, "bfloat16").generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
    clear = 0
    for prompt, out in zip(prompts, got):
        assert len(out) == 12
        clear += _greedy_follows_plain(config, weights, prompt, out, rel=3e-2)
    assert clear >= 12                                   # of 36 places: enough of them decide between two tokens


def test_graphs_and_eager_generate_the_same_ids(tmp_path):
    """The reference's own check of its graph path (tools/diff_cudagraph.py:20-68)."""
    from kvcache_b200 import SamplingParams
    folder = make_model_folder(tmp_path, "B", dtype=torch.bfloat16)
    config, _ = read_folder(folder)
    prompts = [random_tokens(config["vocab_size"], n, 90 + n) for n in (6, 48, 64, 11)]
    params = SamplingParams(max_new_tokens=48, ignore_eos=True)
    for dtype in ("float32", "bfloat16"):
        eager = _llm(folder, "B", dtype, use_graphs=False, num_pages=128).generate(prompts, params)
        graph = _llm(folder, "B", dtype, use_graphs=True, num_pages=128).generate(prompts, params)
        assert eager == graph


def test_temperature_is_reproducible_and_batch_invariant(tmp_path):
    from kvcache_b200 import SamplingParams
    folder = make_model_folder(tmp_path, "B", dtype=torch.bfloat16)
    config, _ = read_folder(folder)
    prompts = [random_tokens(config["vocab_size"], n, 50 + n) for n in (1, 9, 24, 40, 63)]
    params = [SamplingParams(max_new_tokens=12, temperature=0.7, seed=100 + i, ignore_eos=True) for i in range(5)]
    first = _llm(folder, "B", "float32").generate(prompts, params)
    again = _llm(folder, "B", "float32", max_running=2, chunk_size=7, max_tokens_per_step=20).generate(prompts, params)
    assert first == again
    assert len({tuple(o) for o in first}) > 1


def test_optimistic_admission_with_preemption_gives_the_same_ids(tmp_path):
    from kvcache_b200 import SamplingParams
    folder = make_model_folder(tmp_path, "B", dtype=torch.bfloat16)
    config, weights = read_folder(folder)
    prompts = [random_tokens(config["vocab_size"], n, 60 + n) for n in (20, 21, 22)]
    params = SamplingParams(max_new_tokens=20, ignore_eos=True)
    llm = _llm(folder, "B", "float32", num_pages=11, admission="optimistic")    # 88 tokens for 3 x 42
    got = llm.generate(prompts, params)
    assert llm.last_stats.preemptions >= 1
    for prompt, out in zip(prompts, got):
        assert out == greedy_generate(config, weights, prompt, 20)


def test_command_lines(tmp_path):
    folder = make_model_folder(tmp_path, "A", dtype=torch.bfloat16)
    config, weights = read_folder(folder)
    prompts = [random_tokens(config["vocab_size"], n, 95 + n) for n in (7, 19)]
    text = f"{len(prompts)}\n" + "".join(f"6 {' '.join(map(str, p))}\n" for p in prompts)
    serve = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qwen_serve"), folder, "--dtype", "float32",
                            "--ignore-eos"], input=text, capture_output=True, text=True, timeout=600)
    assert serve.returncode == 0, serve.stderr[-2000:]
    lines = [[int(t) for t in l.split()] for l in serve.stdout.splitlines() if l.strip()]
    assert lines == [greedy_generate(config, weights, p, 6) for p in prompts]
    assert "[serve] 2 requests" in serve.stderr and "[serve] done." in serve.stderr
    infer = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qwen_infer"), folder, "6", "--dtype", "float32"],
                           input=" ".join(map(str, prompts[0])), capture_output=True, text=True, timeout=600)
    assert infer.returncode == 0, infer.stderr[-2000:]
    assert [int(t) for t in infer.stdout.split()] == lines[0]
    assert "[infer] prompt_len=7 max_new=6" in infer.stderr and "[bench]" in infer.stderr
