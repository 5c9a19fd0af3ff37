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
NAMES = ["A", "B", "C"]      # (configuration D, head size 64, is met in the tests of its kernels and batches)
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
def test_portions_replayed_from_graphs_equal_eager_launches(tmp_path, kernels, dtype):
    """A step that brings one portion of one prompt is captured when its (length, lengths of the work lists)
    have come often enough (here: twice), and replayed from then on; the logits are those of eager launches, bit for bit,
    also when the same graph serves another request at other pages."""
    runner, config, weights = _runner(tmp_path, kernels, "B", dtype)
    tokens = random_tokens(config["vocab_size"], 101, 16)
    sizes = [20, 20, 20, 20, 21]
    eager = replay_modes.portions(runner, tokens, sizes)
    runner.use_graphs, runner.graph_after_sightings = True, 2
    first = replay_modes.portions(runner, tokens, sizes)
    other = random_tokens(config["vocab_size"], 101, 17)
    runner.use_graphs = False
    eager_other = replay_modes.portions(runner, other, sizes)
    runner.use_graphs = True
    again = replay_modes.portions(runner, other, sizes)
    assert len(runner._graphs) >= 1 and len(sizes) <= runner.graph_replays < 2 * len(sizes)
    assert torch.equal(first, eager) and torch.equal(again, eager_other)
    assert_close(first, logits_of(config, weights, tokens), REL[dtype])
    kernels.check_errors()


def test_mixed_steps_split_into_replayed_parts_sample_the_same_tokens(tmp_path, kernels):
    """With graphs, a sampling step that mixes decoded tokens with portions of prompts runs as the decoded tokens
    and then each portion by itself.  The sampled tokens (float32, greedy, fed with the same ids either way) are
    those of the step run whole, in the order of the entries; the decoded tokens' ids come from the step before,
    on the device; a split step that lacks pages fails before any part of it ran."""
    from kvcache_b200.cache.pages import OutOfPages
    from kvcache_b200.engine.runner import StepEntry
    runner, config, weights = _runner(tmp_path, kernels, "B", "float32", num_pages=40)
    vocab = config["vocab_size"]
    prompts = [random_tokens(vocab, n, 30 + n) for n in (21, 34, 70)]
    greedy = (0.0, 0, 0)
    runner.graph_after_sightings = 2

    def run(split):
        runner.use_graphs, runner.split_mixed_steps = True, split
        cache, seen = runner.cache, []
        slots = [cache.admit() for _ in prompts]
        for slot, prompt in zip(slots[:2], prompts[:2]):
            _, tokens = runner.step([StepEntry(slot, prompt, [len(prompt) - 1], greedy)], sample=True)
            seen.append(tokens.tolist())
        _, tokens = runner.step([StepEntry(s, [0], [0], greedy, token_from_last=0) for s in slots[:2]], sample=True)
        # decoded tokens (their ids: what the step before sampled, still on the device) beside portions of the third
        for start in range(0, 60, 20):
            entries = [StepEntry(s, [0], [0], greedy, token_from_last=i) for i, s in enumerate(slots[:2])]
            entries.append(StepEntry(slots[2], prompts[2][start:start + 20], [19], greedy))
            _, tokens = runner.step(entries, sample=True)
            seen.append(tokens.tolist())
            assert len(seen[-1]) == 3
        lengths = [int(cache.lengths[s]) for s in slots]
        for s in slots:
            cache.release(s)
        return seen, lengths

    replays = runner.graph_replays
    whole, lengths = run(False)
    whole_replays = runner.graph_replays - replays
    run(True)                                                 # the portions' shapes are seen once ...
    replays = runner.graph_replays
    split, lengths_split = run(True)                          # ... and replayed at the second time
    assert split == whole and lengths == lengths_split == [25, 38, 60]
    assert runner.graph_replays - replays > whole_replays
    # the plain implementation agrees on the third prompt's tokens (its logits are those of the prompt so far)
    for start, tokens in zip(range(0, 60, 20), whole[2:]):
        assert tokens[2] == int(logits_of(config, weights, prompts[2][:start + 20])[-1].argmax())
    # 40 pages of 8: two requests hold 2 x 38 pages' worth already, the third wants more than is left
    slots = [runner.cache.admit() for _ in range(3)]
    long = random_tokens(vocab, 150, 9)
    runner.step([StepEntry(slots[0], long, [149], greedy)], sample=True)
    runner.step([StepEntry(slots[1], long, [149], greedy)], sample=True)
    before = [int(runner.cache.lengths[s]) for s in slots]
    with pytest.raises(OutOfPages):
        runner.step([StepEntry(slots[0], [1], [0], greedy), StepEntry(slots[2], long[:40], [39], greedy)], sample=True)
    assert [int(runner.cache.lengths[s]) for s in slots] == before
    kernels.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
def test_head_size_64_long_prompt_and_decoding(tmp_path, kernels, dtype):
    """Configuration D has the head size of the benchmarked model (64; seven query heads on one kv head; its second
    layer windowed), so in bfloat16 a prompt of 700 tokens goes through the tensor-memory prefill kernel and
    decoding through the TMA decode kernel - whole, in portions of which the first is long, and with the last
    32 tokens one by one - against the plain implementation."""
    runner, config, weights = _runner(tmp_path, kernels, "D", dtype, num_pages=96, max_tokens_per_step=1024,
                                      max_tokens_per_request=1024)
    tokens = random_tokens(config["vocab_size"], 700, 21)
    want = logits_of(config, weights, tokens)
    assert_close(replay_modes.whole(runner, tokens), want, REL[dtype], "whole")
    assert_close(replay_modes.portions(runner, tokens, [450, 2, 130, 118]), want, REL[dtype], "portions")
    assert_close(replay_modes.last_32_one_by_one(runner, tokens), want[-33:], REL[dtype], "last 32 one by one")
    kernels.check_errors()
    if dtype == "bfloat16":                                  # the kernels this test is about were the ones that ran
        assert kernels._attn_tc[64]._lib is not None and kernels._flash[64]._lib is not None
        assert kernels.decode_merge == "tma" and kernels.tc_attention_min_rows <= 450


def test_decoding_with_rotation_and_append_inside_attention(tmp_path, kernels, request):
    """Decode steps whose attention kernel also adds the biases, rotates queries and keys and appends the new keys
    and values (the engine takes that kernel from a number of requests on; here from one): two requests of
    different lengths decoded side by side for 330 steps - over page and key-tile edges, the second layer's window
    giving pages back behind them - against the plain implementation; then one of them goes on alone."""
    from kvcache_b200.engine.runner import StepEntry
    saved = kernels.fused_rope_min_requests
    request.addfinalizer(lambda: setattr(kernels, "fused_rope_min_requests", saved))
    kernels.fused_rope_min_requests = 1
    runner, config, weights = _runner(tmp_path, kernels, "D", "bfloat16", num_pages=96, max_tokens_per_step=1024,
                                      max_tokens_per_request=1024)
    a, b = random_tokens(config["vocab_size"], 451, 31), random_tokens(config["vocab_size"], 380, 32)
    want_a, want_b = logits_of(config, weights, a), logits_of(config, weights, b)
    sa, sb = runner.cache.admit(), runner.cache.admit()
    runner.step([StepEntry(sa, a[:100], [99]), StepEntry(sb, b[:50], [49])])
    got_a, got_b = [], []
    for i in range(330):
        out = runner.step([StepEntry(sa, a[100 + i:101 + i], [0]), StepEntry(sb, b[50 + i:51 + i], [0])]).clone()
        got_a.append(out[0])
        got_b.append(out[1])
    counts = []
    for i in range(430, 451):
        if i == 441:
            kernels.fused_rope_min_requests = None           # the last ten steps with the separate rotation kernel again
        launches = kernels.launches
        got_a.append(runner.step([StepEntry(sa, a[i:i + 1], [0])]).clone()[0])
        counts.append(kernels.launches - launches)
    assert counts[0] == counts[-1] - len(runner.model.schedule)       # one launch fewer a layer
    assert_close(torch.stack(got_a), want_a[100:], REL["bfloat16"], "the longer request")
    assert_close(torch.stack(got_b), want_b[50:], REL["bfloat16"], "the shorter request")
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
    """The same request alone and beside three others.  In float32 every reduction belongs to one row and runs in
    an order of its own: bit for bit the same.  In bfloat16 the two steps differ in their number of rows (40 and 77),
    for which the library's matrix product may split its sums differently: equal beyond rounding."""
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
    if dtype == "float32":
        assert torch.equal(together, alone)
    else:
        assert_close(together, alone, 2e-2)


@pytest.mark.parametrize("name", ["B", "D"])
def test_bfloat16_rows_do_not_depend_on_the_batch_within_a_kernel_family(tmp_path, kernels, name):
    """bfloat16, steps that stay within one family of kernels (the small-M products that split K by the weight's shape
    alone, attention whose split over the keys follows from the block table's capacity): a request's logits are the
    same bit for bit whether it runs alone or beside others - a short portion alone and beside another, and its decoded
    tokens alone and beside three decoding requests."""
    from kvcache_b200.engine.runner import StepEntry
    runner, config, weights = _runner(tmp_path, kernels, name, "bfloat16")
    V = config["vocab_size"]
    a = random_tokens(V, 12 + 8, 30)
    others = [random_tokens(V, n, 31 + n) for n in (3, 9, 14)]

    def run(beside: bool):
        slots = [runner.cache.admit() for _ in range(4)]
        got = []
        first = [StepEntry(slots[0], a[:12], list(range(12)))]
        if beside:
            first.append(StepEntry(slots[1], others[0], []))                    # 15 rows in all: the same product kernels
        got.append(runner.step(first).clone()[:12])
        if beside:
            runner.step([StepEntry(slots[2], others[1], []), StepEntry(slots[3], others[2][:-8], [])])
        for i in range(8):
            entries = [StepEntry(slots[0], a[12 + i:13 + i], [0])]
            if beside:
                entries = [StepEntry(slots[1], [5 + i], []), entries[0], StepEntry(slots[2], [7 + i], [0]),
                           StepEntry(slots[3], others[2][-8 + i:len(others[2]) - 7 + i], [])]
            out = runner.step(entries).clone()
            got.append(out[0:1])                                                # a's row is the first wanted row in both
        for s in slots:
            runner.cache.release(s)
        return torch.cat(got)
    alone, beside = run(False), run(True)
    assert torch.equal(alone, beside)
    assert_close(alone, logits_of(config, weights, a), REL["bfloat16"])
    kernels.check_errors()


SHARPEN = {"B": 10.0, "C": 3.0}


def _sharpened_folder(tmp_path, name):
    """A tiny model whose query and key projections are scaled up, so that the softmax of every layer is peaked:
    each row's output hangs on a few keys, often far away, and a key that is lost, doubled or taken from the wrong
    page (a page's edge, a page that was used before, the far edge of a window) moves the logits by far more than
    rounding - with plain random weights attention is nearly uniform and would average such a fault away.
    The factors are chosen so that the plain implementation run in float32 still agrees with itself in float64
    to better than 1e-5 (a sharper model amplifies float32 rounding itself), while changing one token anywhere in
    the prompt moves the last logits by 5e-2 or more of their size."""
    factor = SHARPEN[name]
    from safetensors.torch import load_file, save_file
    import os
    folder = make_model_folder(tmp_path, name, seed=5, dtype=torch.bfloat16)
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    for key in list(tensors):
        if key.endswith("q_proj.weight") or key.endswith("k_proj.weight"):
            tensors[key] = (tensors[key].float() * factor).to(torch.bfloat16)
    save_file(tensors, path)
    return folder


@pytest.mark.parametrize("name", ["B", "C"])
def test_sharp_attention_over_many_pages(tmp_path, kernels, name):
    """float32 only: in bfloat16 the same sharpness amplifies the rounding of activations to the size of the
    effect looked for; the bfloat16 attention kernels meet their far keys and window edges in test_kernels_gpu."""
    dtype = "float32"
    folder = _sharpened_folder(tmp_path, name)
    config, weights = read_folder(folder)
    runner = make_runner(folder, kernels, dtype=dtype, device=DEV, page_size=PAGE_SIZE[name], num_pages=80,
                         max_tokens_per_step=512)
    tokens = random_tokens(config["vocab_size"], 420, 8)
    want = logits_of(config, weights, tokens)
    # The plain model's attention really is peaked: otherwise this test shows nothing.
    for far in (5, 200, 390):
        probe = logits_of(config, weights, tokens[:far] + [(tokens[far] + 1) % config["vocab_size"]] + tokens[far + 1:])
        assert (probe[-1] - want[-1]).abs().max() > 2e-2 * want[-1].abs().max()
    rel = 1e-4
    assert_close(replay_modes.whole(runner, tokens), want, rel, "whole")
    assert_close(replay_modes.last_32_one_by_one(runner, tokens), want[-33:], rel, "one by one")
    assert_close(replay_modes.portions(runner, tokens, [130, 2, 61, 7, 64, 3, 120, 33]), want, rel, "portions")
    # Two requests side by side after the pages above were given back: every page they get was used before.
    other = random_tokens(config["vocab_size"], 200, 9)
    from kvcache_b200.engine.runner import StepEntry
    a, b = runner.cache.admit(), runner.cache.admit()
    got_a, got_b = [], []
    at_a = at_b = 0
    for na, nb in [(100, 1), (1, 150), (200, 2), (1, 47), (118, 0)]:
        entries, parts = [], []
        if na:
            entries.append(StepEntry(a, tokens[at_a:at_a + na], list(range(na)))); parts.append(("a", na)); at_a += na
        if nb:
            entries.append(StepEntry(b, other[at_b:at_b + nb], list(range(nb)))); parts.append(("b", nb)); at_b += nb
        out = runner.step(entries).clone()
        at = 0
        for who, n in parts:
            (got_a if who == "a" else got_b).append(out[at:at + n]); at += n
    assert at_a == 420 and at_b == 200
    assert_close(torch.cat(got_a), want, rel, "mixed a")
    assert_close(torch.cat(got_b), logits_of(config, weights, other), rel, "mixed b")
    kernels.check_errors()
