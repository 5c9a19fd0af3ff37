"""The plain implementation and the engine held to kimxinw/kvcache's own execution.

The reference's model code is CUDA with one model's sizes compiled in; on a GPU its programs run as
they are (baseline/reference_arm.py compiles them, unmodified, for sm_100a).  Here its `qwen_infer`
generates greedily from four prompts with a random model of exactly those sizes - untied head, so that
embedding and output matrix are told apart - and every token it chose is compared with the plain
implementation's choice at that place, given the same tokens before it (tools/run_serve.py:45-49 is the
model for comparing ids).  The reference computes in float16 and prints ids only, so a place counts
where the plain implementation's first choice leads its second by more than MARGIN of the largest
logit: float16 rounding (2^-11 per stored value, some hundred stored values deep) moves a logit by
about a thousandth of the largest one, while a wrong pairing of rotated dimensions, head mapping,
norm, bias or activation moves them by as much as they are large.  This pins the reading of those
formulas in tests/plain_qwen2.py to what the reference computes.
"""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))

MARGIN = 2e-2
NEW_TOKENS = 12
PROMPT_LENGTHS = (5, 17, 33, 70)

REFERENCE_SHAPED = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 896, "num_hidden_layers": 24,
    "num_attention_heads": 14, "num_key_value_heads": 2, "intermediate_size": 4864, "vocab_size": 151936,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": False, "max_position_embeddings": 256,
    "hidden_act": "silu", "use_sliding_window": False, "sliding_window": None, "max_window_layers": 24,
}


@pytest.fixture(scope="module")
def anchored(tmp_path_factory):
    import reference_arm as ra
    try:
        ra.programs()
    except ra.ReferenceUnavailable as exc:
        pytest.skip(f"the reference's programs are not available: {exc}")
    import kvcache_b200  # noqa: F401
    from kvcache_b200.config import config_from_dict
    from kvcache_b200.weights import write_random_model
    from plain_qwen2 import logits_of, read_folder
    tmp = tmp_path_factory.mktemp("reference_anchor")
    folder = write_random_model(os.path.join(str(tmp), "model"), config_from_dict(REFERENCE_SHAPED), seed=11, dtype=torch.bfloat16)
    weights_dir = ra.export_weights(folder, os.path.join(str(tmp), "reference_weights"))
    g = torch.Generator().manual_seed(12)
    cases = []
    config, weights = read_folder(folder, torch.float32)
    for length in PROMPT_LENGTHS:
        prompt = torch.randint(0, REFERENCE_SHAPED["vocab_size"], (length,), generator=g).tolist()
        ids, _ = ra.run_infer(weights_dir, prompt, NEW_TOKENS, graph=False)
        assert len(ids) == NEW_TOKENS
        plain = logits_of(config, weights, prompt + ids[:-1])[length - 1:]          # the rows that chose ids[0], ids[1], ...
        cases.append((prompt, ids, plain))
    return ra, folder, weights_dir, cases


def _clear_places(plain):
    top = torch.topk(plain, 2, dim=-1)
    margin = top.values[:, 0] - top.values[:, 1]
    return margin > MARGIN * plain.abs().max(), top.indices[:, 0]


@pytest.mark.gpu
def test_reference_tokens_are_the_plain_implementations_choice(anchored):
    _, _, _, cases = anchored
    checked = 0
    for prompt, ids, plain in cases:
        clear, choice = _clear_places(plain)
        for i, tok in enumerate(ids):
            if clear[i]:
                checked += 1
                assert tok == int(choice[i]), (f"prompt of {len(prompt)} tokens, generated token {i}: the reference chose {tok}, "
                                               f"the plain implementation {int(choice[i])}")
    assert checked >= len(cases) * NEW_TOKENS // 2, f"only {checked} places had a clear first choice"


@pytest.mark.gpu
def test_reference_graph_decode_equals_eager(anchored):
    """The reference's own claim (README.md:150): CUDA-graph and eager decoding generate the same ids."""
    ra, _, weights_dir, cases = anchored
    prompt, ids, _ = cases[1]
    graph_ids, _ = ra.run_infer(weights_dir, prompt, NEW_TOKENS, graph=True)
    assert graph_ids == ids


@pytest.mark.gpu
def test_reference_serve_equals_infer(anchored):
    """Batched through `qwen_serve`, each request gets the ids `qwen_infer` gave it alone
    (the check of tools/run_serve.py:45-49), up to an end token of the reference's two."""
    ra, _, weights_dir, cases = anchored
    served, _, _ = ra.run_serve(weights_dir, [(NEW_TOKENS, prompt) for prompt, _, _ in cases])
    for (prompt, ids, _), got in zip(cases, served):
        assert got == ids[:len(got)] and (len(got) == NEW_TOKENS or got[-1] in ra.SERVE_EOS)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_engine_chooses_the_references_tokens(anchored, dtype):
    """The engine, given the reference's own tokens, makes the reference's choice wherever the choice is clear."""
    from kvcache_b200.config.options import EngineOptions
    from kvcache_b200.engine.core import EngineCore
    from kvcache_b200.engine.runner import StepEntry
    _, folder, _, cases = anchored
    core = EngineCore(folder, EngineOptions(dtype=dtype, page_size=16, max_cached_tokens=256, max_running=1,
                                            max_tokens_per_step=128, use_graphs=False))
    checked = 0
    for prompt, ids, plain in cases:
        slot = core.cache.admit()
        tokens = prompt + ids[:-1]
        logits = core.runner.step([StepEntry(slot, tokens, list(range(len(prompt) - 1, len(tokens))))])
        choice = torch.argmax(logits, dim=-1).cpu()
        core.cache.release(slot)
        clear, _ = _clear_places(plain)
        for i, tok in enumerate(ids):
            if clear[i]:
                checked += 1
                assert tok == int(choice[i])
    core.kernels.check_errors()
    assert checked >= len(cases) * NEW_TOKENS // 2
