"""The step function: one batch of (request, its next tokens) through the model, from the cache.

The reference has two forwards - a whole prompt of one sequence
(apps/qwen_serve.cu:90-124) and one token for each running sequence (:127-175) -
and rebuilds and copies five metadata arrays per step (:129-147).  Here one
`step` takes any mix of prompt portions and single decoded tokens, cut anywhere,
packs the step's metadata into one host buffer, copies it once, runs only the rows
it was given and returns float32 logits at the wanted places.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..parts.base import StepBatch
from ..parts.model import DecoderModel
from .workspace import Workspace


@dataclass
class StepEntry:
    """One request's share of a step: its slot, its next tokens, and the places among
    these tokens whose logits are wanted."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


def _align4(n: int) -> int:
    return (n + 3) & ~3


class StepLayout:
    """Where each array of a step's metadata lies in the packed int32 buffer."""

    def __init__(self, T: int, S: int, R: int, table_width: int, num_groups: int):
        self.T, self.S, self.R = T, S, R
        self.table_width, self.num_groups = table_width, num_groups
        offset = 0
        self.offsets = {}
        for name, count in (("token_ids", T), ("positions", T), ("row_segment", T), ("seg_q_start", S),
                            ("seg_q_len", S), ("seg_kv_len", S), ("seg_slot", S), ("wanted_rows", R)):
            self.offsets[name] = (offset, count)
            offset += _align4(count)
        self.table_offsets = []
        for _ in range(num_groups):
            self.table_offsets.append(offset)
            offset += _align4(S * table_width)
        self.total = offset

    def view(self, buf, name: str):
        begin, count = self.offsets[name]
        return buf[begin:begin + count]

    def table(self, buf, group: int):
        begin = self.table_offsets[group]
        return buf[begin:begin + self.S * self.table_width].view(self.S, self.table_width) \
            if isinstance(buf, torch.Tensor) else buf[begin:begin + self.S * self.table_width].reshape(self.S, self.table_width)


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager, kernels, *, max_tokens_per_step: int,
                 max_segments: Optional[int] = None):
        self.model, self.cache, self.kernels = model, cache, kernels
        self.device = model.device
        self.max_tokens = max_tokens_per_step
        self.max_segments = max_segments or cache.max_slots
        self.workspace = Workspace(self.device)
        width = cache.max_pages_per_request
        groups = len(cache.groups)
        capacity = StepLayout(self.max_tokens, self.max_segments, self.max_tokens, width, groups).total
        self._meta_device = torch.zeros(capacity, dtype=torch.int32, device=self.device)
        self._on_cuda = self.device.type == "cuda"
        ring = 4 if self._on_cuda else 1
        self._staging = [torch.zeros(capacity, dtype=torch.int32, pin_memory=self._on_cuda) for _ in range(ring)]
        self._staging_events = [None] * ring
        self._ring = 0
        self.steps_run = 0

    # ---- metadata ----------------------------------------------------------
    def _next_staging(self):
        i = self._ring
        self._ring = (self._ring + 1) % len(self._staging)
        event = self._staging_events[i]
        if event is not None:
            event.synchronize()
        return i, self._staging[i]

    def prepare(self, entries: Sequence[StepEntry]) -> Tuple[StepBatch, "object"]:
        """Extends the cache for the entries, packs and uploads the step's metadata."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        counts = [len(e.tokens) for e in entries]
        T, S = sum(counts), len(entries)
        if S > self.max_segments:
            raise ValueError(f"{S} requests in one step; the runner was made for {self.max_segments}")
        if T > self.max_tokens:
            raise ValueError(f"{T} tokens in one step; the runner was made for {self.max_tokens}")
        for e, n in zip(entries, counts):
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"wanted place {w} is outside the {n} tokens the request brings")
        starts = [self.cache.length(e.slot) for e in entries]
        self.cache.extend([(e.slot, n) for e, n in zip(entries, counts)])   # raises OutOfPages before any change

        R = sum(len(e.want) for e in entries)
        layout = StepLayout(T, S, R, self.cache.max_pages_per_request, len(self.cache.groups))
        index, staging = self._next_staging()
        host = staging.numpy()
        counts_np = np.asarray(counts, dtype=np.int32)
        starts_np = np.asarray(starts, dtype=np.int32)
        q_start = np.zeros(S, dtype=np.int32)
        np.cumsum(counts_np[:-1], out=q_start[1:])
        layout.view(host, "token_ids")[:] = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
        row_segment = np.repeat(np.arange(S, dtype=np.int32), counts_np)
        layout.view(host, "row_segment")[:] = row_segment
        layout.view(host, "positions")[:] = np.arange(T, dtype=np.int32) - q_start[row_segment] + starts_np[row_segment]
        layout.view(host, "seg_q_start")[:] = q_start
        layout.view(host, "seg_q_len")[:] = counts_np
        layout.view(host, "seg_kv_len")[:] = starts_np + counts_np
        slots = [e.slot for e in entries]
        layout.view(host, "seg_slot")[:] = np.asarray(slots, dtype=np.int32)
        if R:
            layout.view(host, "wanted_rows")[:] = np.concatenate(
                [q_start[i] + np.asarray(e.want, dtype=np.int32) for i, e in enumerate(entries) if len(e.want)])
        for g in range(len(self.cache.groups)):
            layout.table(host, g)[:] = self.cache.table_rows(g, slots)

        dev = self._meta_device
        dev[:layout.total].copy_(staging[:layout.total], non_blocking=True)
        if self._on_cuda:
            event = torch.cuda.Event()
            event.record()
            self._staging_events[index] = event
        batch = StepBatch(
            num_tokens=T, num_segments=S, num_wanted=R,
            token_ids=layout.view(dev, "token_ids"), positions=layout.view(dev, "positions"),
            row_segment=layout.view(dev, "row_segment"), seg_q_start=layout.view(dev, "seg_q_start"),
            seg_q_len=layout.view(dev, "seg_q_len"), seg_kv_len=layout.view(dev, "seg_kv_len"),
            seg_slot=layout.view(dev, "seg_slot"), wanted_rows=layout.view(dev, "wanted_rows"),
            max_q_len=int(counts_np.max()), max_kv_len=int((starts_np + counts_np).max()),
            host={"counts": counts_np, "starts": starts_np, "q_start": q_start, "slots": slots})
        view = self.cache.step_view([layout.table(dev, g) for g in range(len(self.cache.groups))])
        return batch, view

    # ---- the step ----------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs the entries as one batch; returns float32 logits [wanted places, vocab] in the
        order of the entries and of their `want` lists.  The tensor is a view of a buffer
        the next step overwrites."""
        batch, view = self.prepare(entries)
        logits = self.model.forward(batch, self.kernels, self.workspace, view)
        self.steps_run += 1
        return logits
