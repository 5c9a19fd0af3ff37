"""The ways of cutting and batching that every backend is replayed in.  Each function runs
requests through a runner's step function and returns {request: logits of all its places},
to be compared with the plain implementation's whole-sequence logits."""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from kvcache_b200.engine.runner import StepEntry


def whole(runner, tokens: Sequence[int]) -> torch.Tensor:
    slot = runner.cache.admit()
    out = runner.step([StepEntry(slot, tokens, list(range(len(tokens))))]).clone()
    runner.cache.release(slot)
    return out


def last_32_one_by_one(runner, tokens: Sequence[int]) -> torch.Tensor:
    """Most of it in one step, the last 32 tokens one by one; logits of the last 33 places."""
    slot = runner.cache.admit()
    head = len(tokens) - 32
    got = [runner.step([StepEntry(slot, tokens[:head], [head - 1])]).clone()]
    for i in range(head, len(tokens)):
        got.append(runner.step([StepEntry(slot, tokens[i:i + 1], [0])]).clone())
    runner.cache.release(slot)
    return torch.cat(got)


def portions(runner, tokens: Sequence[int], sizes: Sequence[int]) -> torch.Tensor:
    slot = runner.cache.admit()
    got, at = [], 0
    for size in sizes:
        piece = tokens[at:at + size]
        if not piece:
            break
        got.append(runner.step([StepEntry(slot, piece, list(range(len(piece))))]).clone())
        at += len(piece)
    assert at == len(tokens), "the sizes must cover the sequence"
    runner.cache.release(slot)
    return torch.cat(got)


MIXED_LENGTHS = [("a", 60), ("b", 37), ("c", 64), ("d", 45), ("e", 50)]
# Up to four live requests; portions of some beside single tokens of others; a and b end and
# d and e take their pages.
MIXED_PLAN = [
    [("a", 30), ("b", 5)],
    [("a", 1), ("b", 20), ("c", 33)],
    [("a", 1), ("b", 12), ("c", 2)],
    [("a", 28), ("c", 29)],
    "end a", "end b",
    [("d", 45), ("e", 7), ("c", 0)],
    [("e", 2)],
    "end c",
    [("e", 41)],
]


def mixed_pool_tokens() -> int:
    """Tokens the pool must hold for MIXED_PLAN, each request rounded up to 64."""
    return 64 * 3 + 64


def mixed(runner, seqs: Dict[str, List[int]]) -> Dict[str, torch.Tensor]:
    slots, done = {}, {k: 0 for k in seqs}
    got = {k: [] for k in seqs}
    for item in MIXED_PLAN:
        if isinstance(item, str):
            runner.cache.release(slots.pop(item.split()[1]))
            continue
        parts = [(k, n) for k, n in item if n > 0]
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
    for k in list(slots):
        runner.cache.release(slots.pop(k))
    assert runner.cache.used_pages() == 0
    for k in seqs:
        assert done[k] == len(seqs[k]), k
    return {k: torch.cat(v) for k, v in got.items()}
