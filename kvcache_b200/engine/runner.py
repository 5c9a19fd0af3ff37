"""The step function: one batch of (request, its next tokens) through the model, from the cache.

The reference has two forwards - a whole prompt of one sequence
(apps/qwen_serve.cu:90-124) and one token for each running sequence (:127-175) -
and rebuilds and copies five metadata arrays per step (:129-147).  Here one
`step` takes any mix of prompt portions and single decoded tokens, cut anywhere,
packs the step's metadata into one host buffer, copies it once, runs only the rows
it was given and returns float32 logits at the wanted places (and, if asked, the
tokens sampled from them on the device).

A step in which every request brings exactly one token and wants its logits is
replayed from a CUDA graph captured for that batch size, as the reference's
qwen_infer captures its one-token forward (apps/qwen_infer.cu:135-208); what
changes between replays - ids, positions, block tables, sampling parameters -
lies in the metadata buffer at fixed addresses.
"""
from __future__ import annotations

import contextlib

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..parts.base import StepBatch, StepPlan, StepPlanner
from ..parts.model import DecoderModel
from .workspace import Workspace


@dataclass
class StepEntry:
    """One request's share of a step: its slot, its next tokens, the places among these
    tokens whose logits are wanted, and how tokens are sampled at those places
    (temperature, seed, tokens sampled so far); None samples greedily."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()
    sampling: Optional[Tuple[float, int, int]] = None
    token_from_last: int = -1      # >= 0: the entry's single token is the previous step's sampled token at this index


def _align4(n: int) -> int:
    return (n + 3) & ~3


class StepLayout:
    """Where each array of a step's metadata lies in the packed int32 buffer: the step's own arrays, then the
    lists of every planner (sized by the planner for T tokens in S segments), then the block-table rows."""

    SECTIONS = (("token_ids", "T", 1), ("positions", "T", 1), ("row_segment", "T", 1), ("seg_q_start", "S", 1),
                ("seg_q_len", "S", 1), ("seg_kv_len", "S", 1), ("seg_slot", "S", 1), ("wanted_rows", "R", 1),
                ("sample_temperature", "R", 1), ("sample_counter", "R", 1), ("sample_seed", "R", 2), ("token_src", "T", 1))

    def __init__(self, T: int, S: int, R: int, table_width: int, num_groups: int, planners: Sequence[StepPlanner] = ()):
        self.T, self.S, self.R = T, S, R
        self.table_width, self.num_groups = table_width, num_groups
        sizes = {"T": T, "S": S, "R": R}
        offset = 0
        self.offsets = {}
        for name, dim, words in self.SECTIONS:
            count = sizes[dim] * words
            self.offsets[name] = (offset, count)
            offset += _align4(count)
        for planner in planners:
            for name, count in planner.sections(T, S).items():
                self.offsets[f"{planner.name}.{name}"] = (offset, count)
                offset += _align4(count)
        self.table_offsets = []
        for _ in range(num_groups):
            self.table_offsets.append(offset)
            offset += _align4(S * table_width)
        self.total = offset
        self._remembered_for = None
        self._remembered = {}
        self._host_views = {}

    def remember(self, buf) -> None:
        """Views of `buf` (the runner's one device buffer) are made once and handed out again: a step asks for two dozen."""
        self._remembered_for = buf
        self._remembered = {}
        self._host_views = {}

    def host_views(self, index: int, host) -> dict:
        """The sections of staging buffer `index` (a numpy array) by name, and its block-table rows under ("table", g)."""
        found = self._host_views.get(index)
        if found is None:
            found = {name: host[begin:begin + count] for name, (begin, count) in self.offsets.items()}
            for g in range(self.num_groups):
                found[("table", g)] = self.table(host, g)
            self._host_views[index] = found
        return found

    def cut(self, buf, name: str, length: int):
        """The first `length` elements of a section of the remembered buffer."""
        key = (name, length)
        found = self._remembered.get(key)
        if found is None:
            found = self._remembered[key] = self.view(buf, name)[:length]
        return found

    def upload_pair(self, index: int, dev, staging):
        """(device slice, pinned slice) of the layout's length for staging buffer `index`."""
        key = ("upload", index)
        found = self._remembered.get(key)
        if found is None:
            found = self._remembered[key] = (dev[:self.total], staging[:self.total])
        return found

    def view(self, buf, name: str):
        if buf is self._remembered_for:
            found = self._remembered.get(name)
            if found is None:
                begin, count = self.offsets[name]
                found = self._remembered[name] = buf[begin:begin + count]
            return found
        begin, count = self.offsets[name]
        return buf[begin:begin + count]

    def table(self, buf, group: int):
        if buf is self._remembered_for and ("table", group) in self._remembered:
            return self._remembered[("table", group)]
        begin = self.table_offsets[group]
        flat = buf[begin:begin + self.S * self.table_width]
        shaped = flat.view(self.S, self.table_width) if isinstance(flat, torch.Tensor) else flat.reshape(self.S, self.table_width)
        if buf is self._remembered_for:
            self._remembered[("table", group)] = shaped
        return shaped


class _DecodeGraph:
    def __init__(self, graph, logits, tokens, launches):
        self.graph, self.logits, self.tokens, self.launches = graph, logits, tokens, launches


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager, kernels, *, max_tokens_per_step: int,
                 max_segments: Optional[int] = None, use_graphs: bool = False):
        self.model, self.cache, self.kernels = model, cache, kernels
        self.device = model.device
        self.max_tokens = max_tokens_per_step
        self.max_segments = max_segments or cache.max_slots
        self.workspace = Workspace(self.device)
        self.graph_workspace = Workspace(self.device, row_capacity=self.max_segments)
        width = cache.max_pages_per_request
        groups = len(cache.groups)
        # Work lists that the kernels of this model's mixers read: planned once a step, packed with the metadata.
        self.planners: List[StepPlanner] = list(model.step_planners(kernels))
        capacity = StepLayout(self.max_tokens, self.max_segments, self.max_tokens, width, groups, self.planners).total
        self._meta_device = torch.zeros(capacity, dtype=torch.int32, device=self.device)
        self._on_cuda = self.device.type == "cuda"
        self.use_graphs = use_graphs and self._on_cuda
        self.split_mixed_steps = True     # see _split
        ring = 4 if self._on_cuda else 1
        self._staging = [torch.zeros(capacity, dtype=torch.int32, pin_memory=self._on_cuda) for _ in range(ring)]
        self._staging_np = [t.numpy() for t in self._staging]
        # Events are made once and recorded again and again, on a stream that is looked up once a step: an event made per
        # use and recorded on "the current stream" costs two stream look-ups of 10-20 us each on the host.
        self._staging_events = [torch.cuda.Event() if self._on_cuda else None for _ in range(ring)]
        self._staging_used = [False] * ring
        self._device_index = (self.device.index or 0) if self._on_cuda else None
        self._ring = 0
        self._graphs: Dict[int, _DecodeGraph] = {}
        self._layouts: Dict[Tuple[int, int, int], StepLayout] = {}
        self._portion_shapes_seen: Dict[tuple, int] = {}
        self._sample_parts = None       # asked of the sampling module when a step first samples
        # Tokens the last sampling step chose, in the order of its wanted places.  The next step may take its
        # input ids from here (StepEntry.token_from_last) without the host ever seeing them.
        self.last_tokens = torch.zeros(max(self.max_segments, 1), dtype=torch.int32, device=self.device)
        self._token_host = [torch.zeros(max(self.max_segments, 1), dtype=torch.int32, pin_memory=self._on_cuda) for _ in range(3)]
        self._token_events = [torch.cuda.Event() if self._on_cuda else None for _ in range(3)]
        self._token_ring = 0
        self.steps_run = 0
        self.last_h2d_bytes = 0
        self.graph_replays = 0

    # ---- metadata ----------------------------------------------------------
    def _next_staging(self):
        i = self._ring
        self._ring = (self._ring + 1) % len(self._staging)
        if self._staging_used[i]:
            self._staging_events[i].synchronize()
        return i, self._staging[i]

    def current_stream(self):
        """The stream the step's work goes to (the caller's current one), as an object that events can be recorded on."""
        return torch.cuda.current_stream(self._device_index) if self._on_cuda else None

    def prepare(self, entries: Sequence[StepEntry]):
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
        layout = self._layouts.get((T, S, R))
        if layout is None:
            if len(self._layouts) > 4096:
                self._layouts.clear()
            layout = self._layouts[(T, S, R)] = StepLayout(T, S, R, self.cache.max_pages_per_request, len(self.cache.groups),
                                                           self.planners)
            layout.remember(self._meta_device)
        index, staging = self._next_staging()
        hv = layout.host_views(index, self._staging_np[index])
        counts_np = np.asarray(counts, dtype=np.int32)
        starts_np = np.asarray(starts, dtype=np.int32)
        q_start = np.zeros(S, dtype=np.int32)
        np.cumsum(counts_np[:-1], out=q_start[1:])
        if T == S:                                   # one token per request: no concatenation needed
            hv["token_ids"][:] = [max(e.tokens[0], 0) for e in entries]
            hv["token_src"][:] = [e.token_from_last for e in entries]
            row_segment = np.arange(S, dtype=np.int32)
            hv["positions"][:] = starts_np
        elif S == 1:                                 # one portion of one prompt
            if entries[0].token_from_last >= 0:
                raise ValueError("token_from_last applies to an entry of one token")
            np.maximum(np.asarray(entries[0].tokens, dtype=np.int32), 0, out=hv["token_ids"])
            hv["token_src"][:] = -1
            row_segment = 0
            hv["positions"][:] = np.arange(starts[0], starts[0] + T, dtype=np.int32)
        else:
            hv["token_ids"][:] = np.maximum(np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries]), 0)
            src = hv["token_src"]
            src[:] = -1
            for i, e in enumerate(entries):
                if e.token_from_last >= 0:
                    if counts[i] != 1:
                        raise ValueError("token_from_last applies to an entry of one token")
                    src[q_start[i]] = e.token_from_last
            row_segment = np.repeat(np.arange(S, dtype=np.int32), counts_np)
            hv["positions"][:] = np.arange(T, dtype=np.int32) - q_start[row_segment] + starts_np[row_segment]
        hv["row_segment"][:] = row_segment
        hv["seg_q_start"][:] = q_start
        hv["seg_q_len"][:] = counts_np
        hv["seg_kv_len"][:] = starts_np + counts_np
        slots = [e.slot for e in entries]
        hv["seg_slot"][:] = slots
        if R:
            wanted, temps, counters, seeds = [], [], [], []
            for i, e in enumerate(entries):
                for w in e.want:
                    wanted.append(q_start[i] + w)
                    t, seed, counter = e.sampling if e.sampling is not None else (0.0, 0, 0)
                    temps.append(t)
                    counters.append(counter)
                    seeds.append(seed & 0x7FFFFFFFFFFFFFFF)
            hv["wanted_rows"][:] = wanted
            hv["sample_temperature"].view(np.float32)[:] = temps
            hv["sample_counter"][:] = counters
            hv["sample_seed"].view(np.int64)[:] = seeds
        for g in range(len(self.cache.groups)):
            hv[("table", g)][:] = self.cache.table_rows(g, slots)
        planned = []
        for planner in self.planners:
            arrays, plan_counts = planner.plan(starts_np, counts_np)
            for name, array in arrays.items():
                if len(array):
                    hv[f"{planner.name}.{name}"][:len(array)] = array
            planned.append((planner.name, {name: len(array) for name, array in arrays.items()}, plan_counts))

        dev = self._meta_device
        there, here = layout.upload_pair(index, dev, staging)
        there.copy_(here, non_blocking=True)
        self.last_h2d_bytes = layout.total * 4
        if self._on_cuda:
            self._staging_events[index].record(self.current_stream())
            self._staging_used[index] = True
        batch = StepBatch(
            num_tokens=T, num_segments=S, num_wanted=R,
            token_ids=layout.view(dev, "token_ids"), positions=layout.view(dev, "positions"),
            row_segment=layout.view(dev, "row_segment"), seg_q_start=layout.view(dev, "seg_q_start"),
            seg_q_len=layout.view(dev, "seg_q_len"), seg_kv_len=layout.view(dev, "seg_kv_len"),
            seg_slot=layout.view(dev, "seg_slot"), wanted_rows=layout.view(dev, "wanted_rows"),
            token_src=layout.view(dev, "token_src"), last_tokens=self.last_tokens,
            plans={name: StepPlan({key: layout.cut(dev, f"{name}.{key}", length) for key, length in lengths.items()}, plan_counts)
                   for name, lengths, plan_counts in planned},
            max_q_len=max(counts), max_kv_len=max(s + c for s, c in zip(starts, counts)),
            host={"counts": counts_np, "starts": starts_np, "q_start": q_start, "slots": slots})
        view = self.cache.step_view([layout.table(dev, g) for g in range(len(self.cache.groups))])
        return batch, view, layout

    # ---- the step ----------------------------------------------------------
    def _sample(self, logits: torch.Tensor, layout: StepLayout, workspace: Workspace, token_offset: int = 0) -> torch.Tensor:
        R = logits.shape[0]
        dev = self._meta_device
        if self._sample_parts is None:
            self._sample_parts = self.kernels.sample_parts(self.model.vocab_size)
        if token_offset + R > self.last_tokens.shape[0]:
            raise ValueError(f"{token_offset + R} places to sample in one step; the runner was made for {self.last_tokens.shape[0]}")
        tokens = self.last_tokens[token_offset:token_offset + R]
        self.kernels.sample(logits, layout.view(dev, "sample_temperature").view(torch.float32),
                            layout.view(dev, "sample_seed").view(torch.int64), layout.view(dev, "sample_counter"), tokens,
                            workspace.buffer("sample.part_val", (R * self._sample_parts,), torch.float32),
                            workspace.buffer("sample.part_idx", (R * self._sample_parts,), torch.int32))
        return tokens

    def _forward(self, batch, view, layout, workspace, sample: bool, token_offset: int = 0):
        scope = getattr(self.kernels, "on_current_stream", None)
        with (scope() if scope is not None else contextlib.nullcontext()):
            logits = self.model.forward(batch, self.kernels, workspace, view)
            tokens = self._sample(logits, layout, workspace, token_offset) if sample and batch.num_wanted else None
        return logits, tokens

    MAX_GRAPHS = 32

    @staticmethod
    def _plan_key(plans) -> tuple:
        return tuple((name, tuple(sorted(counts.items()))) for name, counts in plans)

    def _graph_key(self, batch, sample: bool, token_offset: int = 0):
        """The key under which a step's launches can be replayed, or None.  Two kinds of steps have launches
        that depend on nothing but a few counts: steps of single decoded tokens (the batch size), and steps
        that bring one portion of one prompt (its length and the counts of the planners' work lists, which
        grow with what the prompt has cached).  Everything else - the ids, positions, block tables, the work
        lists themselves - is read from the step's metadata buffer, whose layout these counts fix."""
        if not self.use_graphs:
            return None
        plans = self._plan_key((name, plan.counts) for name, plan in batch.plans.items())
        if sample and batch.num_tokens == batch.num_segments == batch.num_wanted:
            return ("decode", batch.num_tokens, token_offset, plans)
        if batch.num_segments == 1 and batch.num_tokens > 1:
            return ("portion", batch.num_tokens, batch.num_wanted, sample, token_offset, plans)
        return None

    def _portion_key(self, start: int, count: int, wanted: int, sample: bool, token_offset: int):
        """The key `_graph_key` gives a step that brings `count` tokens of one request which has `start` cached."""
        starts, counts = np.asarray([start], dtype=np.int32), np.asarray([count], dtype=np.int32)
        plans = self._plan_key((planner.name, planner.plan(starts, counts)[1]) for planner in self.planners)
        return ("portion", count, wanted, sample, token_offset, plans)

    # Making a graph takes as long as a dozen steps, and prompts of odd lengths bring shapes that never come again: a
    # portion's shape is recorded once it has been seen this often.
    graph_after_sightings = 4

    def _comes_again(self, key, count: bool = True) -> bool:
        """True if `key` has a graph, or has been seen often enough to be given one.  `count`: this call is a
        sighting of its own (False for a second look at a key within one step)."""
        if key in self._graphs:
            return True
        if len(self._portion_shapes_seen) > 4096:
            self._portion_shapes_seen.clear()
        seen = self._portion_shapes_seen.get(key, 0) + (1 if count else 0)
        if count:
            self._portion_shapes_seen[key] = seen
        return seen >= self.graph_after_sightings

    def _graph(self, key, batch, view, layout, sample: bool, token_offset: int = 0):
        """The recorded launches of a step with this key, and whether this call has just made (and thereby run) them.

        A step is recorded the first time its key is wanted: it runs once, launched kernel by kernel, in the graph's
        workspace - that sizes the buffers and is the step's one execution - and then its launches are recorded
        without being run.  The caller replays the graph only from the next step on.  The step therefore takes effect
        exactly once, whatever state its parts keep (keys and values, a mixer's running state, the sampled tokens
        that the step itself may read its ids from).  A part's `forward` is called twice for it on the host; parts
        keep no state of their own on the host."""
        found = self._graphs.pop(key, None)
        if found is not None:
            self._graphs[key] = found                         # the most recently used is the last to go
            return found, False
        if len(self._graphs) >= self.MAX_GRAPHS:
            self._graphs.pop(next(iter(self._graphs)))        # the one not used for longest
        ws = self.graph_workspace
        moved = ws.moved
        self._forward(batch, view, layout, ws, sample, token_offset)
        if ws.moved != moved:
            self._graphs.clear()                              # a buffer moved: graphs that hold its old address go
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        before = self.kernels.launches
        ws.frozen = True
        try:
            with torch.cuda.graph(graph):
                logits, tokens = self._forward(batch, view, layout, ws, sample, token_offset)
        finally:
            ws.frozen = False
        found = _DecodeGraph(graph, logits, tokens, self.kernels.launches - before)
        self._graphs[key] = found
        return found, True

    def read_tokens_async(self, count: int):
        """Starts the copy of the last step's sampled tokens to the host; returns a function that waits for
        it and gives the int32 array.  Steps launched in between do not disturb the copy."""
        index = self._token_ring
        self._token_ring = (self._token_ring + 1) % len(self._token_host)
        host = self._token_host[index]
        host[:count].copy_(self.last_tokens[:count], non_blocking=True)
        if not self._on_cuda:
            return lambda: host[:count].numpy().copy()
        event = self._token_events[index]       # its last use was three reads ago: that copy has long been waited for
        event.record(self.current_stream())

        def wait():
            event.synchronize()
            return host[:count].numpy().copy()
        return wait

    def step(self, entries: Sequence[StepEntry], sample: bool = False):
        """Runs the entries as one batch.  Returns float32 logits [wanted places, vocab] in the
        order of the entries and of their `want` lists - or, with `sample`, the pair
        (logits, int32 tokens sampled at those places, on the device: `last_tokens`).  The
        tensors are views of buffers the next step overwrites."""
        if sample and self.use_graphs and self.split_mixed_steps:
            parts = self._split(entries)
            if parts is not None:
                return self._run_split(entries, parts)
        logits, tokens = self._run(entries, sample, 0)
        self.steps_run += 1
        return (logits, tokens) if sample else logits

    def _run(self, entries: Sequence[StepEntry], sample: bool, token_offset: int, counted: bool = False):
        """`counted`: the step's shape has already been counted as a sighting in this step (by `_split`)."""
        batch, view, layout = self.prepare(entries)
        key = self._graph_key(batch, sample, token_offset)
        if key is not None and key[0] == "portion" and not self._comes_again(key, count=not counted):
            key = None
        if key is not None:
            found, ran = self._graph(key, batch, view, layout, sample, token_offset)
            if not ran:
                found.graph.replay()
                self.graph_replays += 1
            self.kernels.launches += found.launches
            return found.logits, found.tokens
        return self._forward(batch, view, layout, self.workspace, sample, token_offset)

    # A step that mixes decoded tokens with portions of prompts seldom has the shape of a step before it, so it is
    # launched kernel by kernel (about 250 launches, bound by the host).  Where the portions have shapes that came
    # before, it is run as what can be replayed instead: the decoded tokens as one batch, then each portion by itself.
    # Measured at seven decoded tokens beside a portion of 512: 3.1 ms as one batch, 2.2 ms split.  Longer portions keep
    # the step whole: its kernels then take as long as the host needs to launch them.
    SPLIT_MAX_PORTION = 1024

    def _split(self, entries: Sequence[StepEntry]):
        """The entries as [decoded tokens..., one list per portion] if the step mixes both kinds (decoded tokens first,
        as the scheduler orders them) and no portion is long; else None."""
        singles = [e for e in entries if len(e.tokens) == 1 and len(e.want) == 1]
        others = [e for e in entries if not (len(e.tokens) == 1 and len(e.want) == 1)]
        if not singles or not others or list(entries[:len(singles)]) != singles:
            return None
        if any(len(e.tokens) < 2 or len(e.tokens) > self.SPLIT_MAX_PORTION for e in others):
            return None
        # Only portions whose launches can be replayed gain from running alone.
        offset, replayable = len(singles), True
        for e in others:
            key = self._portion_key(self.cache.length(e.slot), len(e.tokens), len(e.want), True, offset)
            replayable = self._comes_again(key) and replayable
            offset += len(e.want)
        return [singles] + [[e] for e in others] if replayable else None

    def _run_split(self, entries: Sequence[StepEntry], parts):
        # All or nothing, as one step would be: every page the whole step needs must be there before any part runs.
        additions = [(e.slot, len(e.tokens)) for e in entries]
        if self.cache.pages_short(additions):
            self.cache.extend(additions)                      # raises the error a whole step would raise
            raise AssertionError("unreachable: extend must have refused")
        offset = 0
        for part in parts:
            self._run(part, True, offset, counted=True)
            offset += sum(len(e.want) for e in part)
        self.steps_run += 1
        return None, self.last_tokens[:offset]
