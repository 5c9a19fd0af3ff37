"""Work lists of the paged-attention kernels: which block of a launch does what.

The tiling belongs to the kernels (csrc/attention_flash.cu, csrc/attention_tc.cu), so the
lists that follow from it are made here, beside the launchers, and not in the step function:
the runner packs whatever a `StepPlanner` hands it.

* `decode_items`: the segments that bring one token (each is one item of the decode kernels).
* `prefill_units`: the segments that bring more, as tiles of 64 query rows cut into units of
  about equal numbers of 64-key tiles (the `mma.sync` prefill kernel), and
* `tc_units`: the same segments as tiles of 128 rows with units of at least 16 key tiles
  (the tensor-memory prefill kernel).

The reference has one block per (query row, head) and no such lists (src/qwen_kernels.cu:146-185).
"""
from __future__ import annotations

import functools
from typing import Dict, Tuple

import numpy as np

from ..parts.base import StepPlanner

PREFILL_TILE_ROWS = 64          # query rows of a prefill attention tile
PREFILL_KEY_TILE = 64           # keys the kernel takes at a time
PREFILL_MAX_UNITS = 16          # most units one tile may be cut into (csrc/attention_flash.cu)
PREFILL_UNITS_WANTED = 256      # about this many units beyond one per tile, however long the prompts
TC_TILE_ROWS = 128              # query rows of a tile of the tensor-memory attention kernel
TC_MIN_KEY_TILES = 16           # a unit of that kernel has at least this many key tiles, unless its tile has fewer


def plan_prefill_units(segments, tile_rows: int = PREFILL_TILE_ROWS, min_key_tiles: int = 4):
    """`_plan_prefill_units`, remembered: a prompt cut into portions of one size, and prompts of one length, bring the
    same segments step after step.  The array that comes back is shared and not to be written."""
    return _plan_prefill_units(tuple(segments), tile_rows, min_key_tiles)


@functools.lru_cache(maxsize=1024)
def _plan_prefill_units(segments, tile_rows: int, min_key_tiles: int):
    """The work list of prefill attention.  `segments`: (segment index, tokens cached before the step, tokens
    it brings) for every segment of more than one token.  A tile is `tile_rows` consecutive rows of a segment;
    a tile whose rows see many keys is cut into units of about equal numbers of key tiles, so that the blocks
    of the grid - one per (unit, head) - all have about the same work although causal tiles do not.  Tiles
    with the most keys come first.
    Returns (int32 array [units, 8]: segment, first row, unit, units of the tile, tile id, first unit of the
    tile, 0, 0; number of tiles)."""
    tiles = []
    for seg, start, count in segments:
        for row0 in range(0, count, tile_rows):
            rows = min(tile_rows, count - row0)
            tiles.append((seg, row0, (start + row0 + rows - 1) // PREFILL_KEY_TILE + 1))
    tiles.sort(key=lambda t: -t[2])
    total = sum(k for _, _, k in tiles)
    per_unit = max(min_key_tiles, -(-total // PREFILL_UNITS_WANTED))
    units = []
    for tile_id, (seg, row0, key_tiles) in enumerate(tiles):
        nsplit = max(1, min(PREFILL_MAX_UNITS, -(-key_tiles // per_unit)))
        first = len(units)
        for split in range(nsplit):
            units.append((seg, row0, split, nsplit, tile_id, first, 0, 0))
    array = np.asarray(units, dtype=np.int32).reshape(-1, 8)
    array.setflags(write=False)
    return array, len(tiles)


class PagedAttentionPlanner(StepPlanner):
    name = "paged_attention"

    def sections(self, num_tokens: int, num_segments: int) -> Dict[str, int]:
        T, S = num_tokens, num_segments
        return {"decode_items": S,
                "prefill_units": 8 * (2 * (T // PREFILL_TILE_ROWS + S) + PREFILL_UNITS_WANTED),
                "tc_units": 8 * (2 * (T // TC_TILE_ROWS + S) + PREFILL_UNITS_WANTED)}

    def plan(self, starts, counts) -> Tuple[Dict[str, np.ndarray], Dict[str, int]]:
        counts = np.asarray(counts)
        S = len(counts)
        if int(counts.sum()) == S:                       # one token per request: every segment is an item, in order
            return ({"decode_items": np.arange(S, dtype=np.int32)},
                    {"decode_items": S, "prefill_units": 0, "prefill_tiles": 0, "tc_units": 0, "tc_tiles": 0})
        single = counts == 1
        items = np.nonzero(single)[0].astype(np.int32)
        longer = [(int(i), int(starts[i]), int(counts[i])) for i in np.nonzero(~single)[0]]
        units, tiles = plan_prefill_units(longer)
        tc_units, tc_tiles = plan_prefill_units(longer, TC_TILE_ROWS, TC_MIN_KEY_TILES)
        return ({"decode_items": items, "prefill_units": units.reshape(-1), "tc_units": tc_units.reshape(-1)},
                {"decode_items": len(items), "prefill_units": len(units), "prefill_tiles": tiles,
                 "tc_units": len(tc_units), "tc_tiles": tc_tiles})
