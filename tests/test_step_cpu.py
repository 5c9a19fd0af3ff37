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


def test_prefill_work_list():
    """Tiles of 64 rows; long tiles are cut into units of about equal numbers of key tiles."""
    from kvcache_b200.kernels.attention_plan import plan_prefill_units
    units, n_tiles = plan_prefill_units([(0, 0, 2048), (3, 100, 2)])
    assert n_tiles == 33 and units.shape[1] == 8
    by_tile = {}
    for seg, row0, split, nsplit, tile_id, first, _, _ in units.tolist():
        by_tile.setdefault(tile_id, []).append((seg, row0, split, nsplit, first))
    assert len(by_tile) == n_tiles
    for tile_id, rows in by_tile.items():
        nsplit = rows[0][3]
        assert [r[2] for r in rows] == list(range(nsplit)) and len({r[4] for r in rows}) == 1
        assert 1 <= nsplit <= 16
    # Tiles with the most keys come first: tile 0 is the prompt's last 64 rows, 32 key tiles in units of 4.
    assert by_tile[0][0][:2] == (0, 2048 - 64) and by_tile[0][0][3] == 8
    assert by_tile[32][0][:2] == (0, 0) and by_tile[32][0][3] == 1 and (3, 0) in {r[0][:2] for r in by_tile.values()}
    # The same prompt in tiles of 128 rows with units of at least 16 key tiles.
    units128, n128 = plan_prefill_units([(0, 0, 2048)], 128, 16)
    assert n128 == 16 and len(units128) == 24 and units128[0].tolist()[:4] == [0, 2048 - 128, 0, 2]
    # However long the prompt, the list stays bounded.
    units, n_tiles = plan_prefill_units([(0, 0, 32768)])
    assert n_tiles == 512 and len(units) <= 2 * 512 + 256


def test_which_mixed_steps_are_run_in_parts(tmp_path):
    """The runner's decision to run a sampling step as its parts (decoded tokens, then each portion alone): only where
    decoded tokens come first and beside portions of at least two and at most SPLIT_MAX_PORTION tokens whose shapes
    have come `graph_after_sightings` times (so that their launches can be replayed); a portion's shape is its length,
    the number of wanted places, the counts of its planners' work lists and where its sampled token goes."""
    from kvcache_b200.engine.runner import StepEntry
    runner, config, _ = _runner(tmp_path, "B", max_tokens_per_step=2048, max_tokens_per_request=2048, num_pages=600)
    runner.graph_after_sightings = 2
    from kvcache_b200.kernels.attention_plan import PagedAttentionPlanner
    runner.planners = [PagedAttentionPlanner()]                         # the work lists of the CUDA kernel set's attention
    a, b, c = (runner.cache.admit() for _ in range(3))
    runner.cache.extend([(a, 40), (b, 7)])
    one = lambda slot: StepEntry(slot, [1], [0], (0.0, 0, 0))
    portion = lambda slot, n, want=True: StepEntry(slot, list(range(n)), [n - 1] if want else [], (0.0, 0, 0))
    assert runner._split([one(a), one(b)]) is None                      # no portion
    assert runner._split([portion(c, 20)]) is None                      # no decoded token
    assert runner._split([one(a), portion(c, 20)]) is None              # the shape's first sighting
    parts = runner._split([one(a), portion(c, 20)])                     # its second
    assert [[e.slot for e in part] for part in parts] == [[a], [c]]
    assert runner._split([one(a), one(b), portion(c, 20)]) is None      # another offset of the sampled token: another shape
    assert runner._split([one(a), portion(c, 20, want=False)]) is None  # nothing wanted: another shape
    assert runner._split([one(a), portion(c, 21)]) is None              # another length
    assert runner._split([portion(c, 20), one(a)]) is None              # decoded tokens must come first
    assert runner._split([one(a), portion(c, 20), one(b)]) is None
    runner._split([one(a), portion(c, 1200)])
    assert runner._split([one(a), portion(c, 1200)]) is None            # too long to gain from it
    assert runner._split([one(a), StepEntry(c, [3], [], None)]) is None  # a one-token portion that wants nothing
    # the same length further into a prompt has longer work lists: another shape, until it has come twice too
    runner.cache.extend([(c, 700)])
    assert runner._split([one(a), portion(c, 20)]) is None
    assert runner._split([one(a), portion(c, 20)]) is not None
    assert runner._portion_key(0, 20, 1, True, 1) != runner._portion_key(700, 20, 1, True, 1)
