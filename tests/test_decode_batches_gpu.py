"""The schedules the benchmark times, held to the plain implementation: 8, 20, 33 and 64 live requests of different
lengths decoded for 40 steps across page edges, replayed from CUDA graphs, with every step's ids taken on the device from
the tokens the step before sampled; and a long portion of a prompt beside decoded tokens in one step.

At these sizes the engine changes kernels - from 16 requests on bias, rotation and append run inside the TMA decode
kernel, 17 to 32 rows go through the weight-streaming tensor-memory product, 33 and more through the library product -
so each case also asserts, from the launch counters, that the kernels it is meant to cover did run.  Shapes: tiny
configuration D (head size 64, 7 query heads on one kv head, a windowed layer) and two layers of the benchmarked
model's layer shape (hidden 896, 14 and 2 heads, intermediate 4,864) with a small vocabulary.
"""
import os
import random

import pytest
import torch

from helpers import assert_close, make_runner, random_tokens
from plain_qwen2 import logits_of, read_folder
from tiny_configs import TINY_D

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REL = {"float32": 1e-4, "bfloat16": 3e-2}
DECODE_STEPS = 40
BENCH_LAYER_SHAPE = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 896, "num_hidden_layers": 2,
    "num_attention_heads": 14, "num_key_value_heads": 2, "intermediate_size": 4864, "vocab_size": 2003,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": True, "max_position_embeddings": 32768,
    "hidden_act": "silu", "use_sliding_window": False, "sliding_window": None, "max_window_layers": 2,
}
FAMILY_15B_LAYER_SHAPE = dict(BENCH_LAYER_SHAPE, hidden_size=1536, num_attention_heads=12, intermediate_size=8960)
SHAPES = {"D": (TINY_D, 32), "0.5B": (BENCH_LAYER_SHAPE, 16), "1.5B": (FAMILY_15B_LAYER_SHAPE, 16)}


@pytest.fixture(scope="module")
def kernels():
    from kvcache_b200.kernels.api import CudaKernels
    return CudaKernels(DEV)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    import kvcache_b200  # noqa: F401
    from kvcache_b200.config import config_from_dict
    from kvcache_b200.weights import write_random_model
    root = tmp_path_factory.mktemp("decode_batches")
    out = {}
    for name, (config, _) in SHAPES.items():
        folder = write_random_model(os.path.join(str(root), name), config_from_dict(config), seed=2, dtype=torch.bfloat16)
        # float32 is plenty for the plain side at these sizes (1e-6 against tolerances of 1e-4 and 3e-2) and four times faster
        out[name] = (folder,) + read_folder(folder, torch.float64 if name == "D" else torch.float32)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("batch", [8, 20, 33, 64])
@pytest.mark.parametrize("shape", ["D", "0.5B"])
def test_decode_batches_of_the_benchmark(folders, kernels, shape, batch, dtype):
    from kvcache_b200.engine.runner import StepEntry
    folder, config, weights = folders[shape]
    page = SHAPES[shape][1]
    rng = random.Random(100 * batch + len(shape))
    lengths = [rng.randint(3, 70) for _ in range(batch)]
    lengths[0], lengths[1] = page - 1, page               # the first decoded token of these lands on a page's edge
    prompts = [random_tokens(config["vocab_size"], n, 1000 + i) for i, n in enumerate(lengths)]
    total = max(lengths) + DECODE_STEPS + 1
    runner = make_runner(folder, kernels, dtype=dtype, device=DEV, page_size=page,
                         num_pages=sum(-(-(n + DECODE_STEPS + 1) // page) for n in lengths) + 2,
                         max_slots=batch, max_tokens_per_step=sum(lengths), max_tokens_per_request=-(-total // page) * page)
    runner.use_graphs = True
    kernels.launch_counts.clear()
    slots = [runner.cache.admit() for _ in range(batch)]
    # All prompts in one step; each samples its first token, which stays on the device.
    logits, tokens = runner.step([StepEntry(s, p, [len(p) - 1], (0.0, 0, 0)) for s, p in zip(slots, prompts)], sample=True)
    got_logits, got_tokens = [logits.clone()], [tokens.clone()]
    for step in range(DECODE_STEPS):
        entries = [StepEntry(s, (0,), (0,), (0.0, 0, step + 1), token_from_last=i) for i, s in enumerate(slots)]
        logits, tokens = runner.step(entries, sample=True)
        got_logits.append(logits.clone())
        got_tokens.append(tokens.clone())
    kernels.check_errors()
    assert runner.graph_replays == DECODE_STEPS - 1       # the first decode step records the launches, the others replay them
    got_logits = torch.stack(got_logits).cpu()            # [steps + 1, batch, V]
    got_tokens = torch.stack(got_tokens).cpu()
    # The sampler's choice is the largest logit, the lowest index among equals.
    assert torch.equal(got_tokens.long(), got_logits.argmax(dim=-1))
    for i, prompt in enumerate(prompts):
        sequence = prompt + got_tokens[:DECODE_STEPS, i].tolist()
        want = logits_of(config, weights, sequence)[len(prompt) - 1:]
        assert_close(got_logits[:, i], want, REL[dtype], f"request {i} of {batch} (prompt of {len(prompt)})")
    counts = kernels.launch_counts
    if dtype == "bfloat16":
        if batch >= 16:
            assert counts["flash_decode_tma_fused"] > 0 and counts["rope_append"] <= config["num_hidden_layers"]
        else:
            assert counts["flash_decode_tma"] > 0
            if shape == "0.5B":                           # (tiny D's widths are no multiples of 32: its products stream through tcgen05)
                assert counts["gemm_skinny"] > 0
                if kernels.fold_norms:
                    # a layer in five launches: norms, adds, bias, rotation and append run inside its products
                    assert counts["gemm_skinny_qkv"] > 0 and counts["gemm_skinny_norm_act"] > 0
                    assert counts["gemm_skinny_residual"] > 0 and counts["rope_append"] <= config["num_hidden_layers"]
        if 17 <= batch <= 32:
            assert counts["gemm_wstream"] > 0
        if batch >= 33:
            assert counts["gemm_library"] > 0
    else:
        assert counts["gemm_simt"] > 0 and counts["attention_generic"] > 0 and not counts["gemm_library"]


@pytest.mark.parametrize("batch", [8, 13])
def test_decode_batches_through_the_folded_chain(folders, kernels, request, batch):
    """The same schedule with the folded forms switched on (a layer in five launches: the norms inside the products after
    them, the adds inside the products before them, bias, rotation and append inside the q/k/v projection)."""
    saved = kernels.fold_norms
    kernels.fold_norms = True
    request.addfinalizer(lambda: setattr(kernels, "fold_norms", saved))
    test_decode_batches_of_the_benchmark(folders, kernels, "0.5B", batch, "bfloat16")


@pytest.mark.parametrize("shape", ["D", "1.5B"])
def test_long_portion_beside_decoded_tokens(folders, kernels, shape):
    """The common mixed step of serving: running requests decode one token each while a waiting request brings a portion
    of some hundred rows that follows a cached prefix.  In bfloat16 the portion goes through the tensor-memory attention
    kernel and the decoded tokens through the TMA decode kernel, both inside one attention call (head sizes 64 and 128)."""
    from kvcache_b200.engine.runner import StepEntry
    folder, config, weights = folders[shape]
    page = SHAPES[shape][1]
    V = config["vocab_size"]
    decoding = [random_tokens(V, n, 50 + i) for i, n in enumerate((51, 131, 300))]
    long_prompt = random_tokens(V, 200 + 450 + 3, 60)
    want_decoded = [logits_of(config, weights, t)[-1:] for t in decoding]
    want_long = logits_of(config, weights, long_prompt[:651])
    for dtype in ("float32", "bfloat16"):
        runner = make_runner(folder, kernels, dtype=dtype, device=DEV, page_size=page, num_pages=1400 // page + 8, max_slots=4,
                             max_tokens_per_step=1024, max_tokens_per_request=1024)
        kernels.launch_counts.clear()
        slots = [runner.cache.admit() for _ in range(4)]
        runner.step([StepEntry(s, t[:-1], []) for s, t in zip(slots[:3], decoding)] + [StepEntry(slots[3], long_prompt[:200], [])])
        before = dict(kernels.launch_counts)
        entries = [StepEntry(slots[0], decoding[0][-1:], [0]), StepEntry(slots[1], decoding[1][-1:], [0]),
                   StepEntry(slots[3], long_prompt[200:650], list(range(450))), StepEntry(slots[2], decoding[2][-1:], [0])]
        out = runner.step(entries).clone()
        kernels.check_errors()
        assert_close(out[0:1], want_decoded[0], REL[dtype], "decoded token 0")
        assert_close(out[1:2], want_decoded[1], REL[dtype], "decoded token 1")
        assert_close(out[2:452], want_long[200:650], REL[dtype], "portion after a cached prefix")
        assert_close(out[452:453], want_decoded[2], REL[dtype], "decoded token 2")
        # and the request goes on decoding from what the mixed step cached
        nxt = runner.step([StepEntry(slots[3], long_prompt[650:651], [0])]).clone()
        assert_close(nxt, want_long[650:651], REL[dtype], "the token after the portion")
        if dtype == "bfloat16":
            ran = {k: v - before.get(k, 0) for k, v in kernels.launch_counts.items()}
            assert ran.get("attention_tc", 0) >= config["num_hidden_layers"] and ran.get("flash_decode_tma", 0) >= config["num_hidden_layers"]
