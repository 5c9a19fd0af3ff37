"""The cache manager: page pools, block tables and state slots for every layer call of a model.

It joins what the reference splits between `KVCacheManager` (pool + tables,
src/include/kv_cache_manager.h:27-92) and the app's own handling
(apps/qwen_serve.cu:85-93, :134-135), and adds groups: cache entries whose keys
and values have the same geometry and reach share one block table and one page id,
as the reference's 24 layers share one (apps/qwen_serve.cu:99-100); entries with
a window form a group of their own and give pages back once the window has passed.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import PagedKVSpec, PagedKVView, TORCH_DTYPES
from ..parts.model import CacheEntry
from .pages import GroupPages, OutOfPages, pages_for
from .slots import SlotAllocator


@dataclass
class CacheGroup:
    spec: PagedKVSpec
    cache_ids: List[int]
    pages: GroupPages
    k_pool: Optional[torch.Tensor] = None     # [entries, pages, kv_heads, page_size, head_dim]
    v_pool: Optional[torch.Tensor] = None


class CacheManager:
    """Host bookkeeping for all groups plus (when `device` is given) the pools themselves.

    A request is admitted into a slot, extended as its tokens are run
    (`extend(slot, start, end)` before the step that runs positions start..end-1)
    and released when it ends.  With `device=None` only the bookkeeping exists,
    which is what the scheduler needs.
    """

    def __init__(self, entries: Sequence[CacheEntry], *, page_size: int, num_pages: int, max_slots: int,
                 max_tokens_per_request: int, dtype: str = "bfloat16", device: Optional[torch.device | str] = None):
        self.page_size, self.num_pages, self.max_slots = page_size, num_pages, max_slots
        self.max_pages_per_request = pages_for(max_tokens_per_request, page_size)
        self.dtype = TORCH_DTYPES[dtype]
        self.device = torch.device(device) if device is not None else None
        self.slots = SlotAllocator(max_slots)
        self.lengths = [0] * max_slots             # a plain list: read several times a step and request, as Python ints
        self.groups: List[CacheGroup] = []
        self.entry_group: Dict[int, Tuple[int, int]] = {}   # cache id -> (group index, index in group)
        self.states: Dict[int, object] = {}      # cache id -> [slots, *shape] tensor, or {name: such a tensor}
        by_spec: Dict[PagedKVSpec, int] = {}
        for cache_id, entry in enumerate(entries):
            if entry.kv is not None:
                if entry.kv not in by_spec:
                    by_spec[entry.kv] = len(self.groups)
                    self.groups.append(CacheGroup(entry.kv, [], GroupPages(
                        num_pages, page_size, max_slots, self.max_pages_per_request, entry.kv.window)))
                g = by_spec[entry.kv]
                self.entry_group[cache_id] = (g, len(self.groups[g].cache_ids))
                self.groups[g].cache_ids.append(cache_id)
            if entry.state is not None and self.device is not None:
                make = lambda spec: torch.zeros((max_slots, *spec.shape), dtype=TORCH_DTYPES[spec.dtype], device=self.device)
                self.states[cache_id] = {name: make(spec) for name, spec in entry.state.items()} \
                    if isinstance(entry.state, dict) else make(entry.state)
        if self.device is not None:
            for group in self.groups:
                shape = (len(group.cache_ids), num_pages, group.spec.num_kv_heads, page_size, group.spec.head_dim)
                group.k_pool = torch.zeros(shape, dtype=self.dtype, device=self.device)
                group.v_pool = torch.zeros(shape, dtype=self.dtype, device=self.device)

    # ---- requests ----------------------------------------------------------
    def admit(self) -> int:
        """Takes a slot for a new request: empty block tables, zeroed state, length 0."""
        slot = self.slots.alloc()
        self.lengths[slot] = 0
        for state in self.state_tensors():
            state[slot].zero_()
        return slot

    def state_tensors(self) -> List[torch.Tensor]:
        """Every per-request state tensor of every cache entry."""
        out: List[torch.Tensor] = []
        for state in self.states.values():
            out.extend(state.values() if isinstance(state, dict) else [state])
        return out

    def length(self, slot: int) -> int:
        """Tokens of the request that steps have run so far (its next position)."""
        return self.lengths[slot]

    def pages_short(self, additions: Sequence[Tuple[int, int]]) -> int:
        """Largest shortfall of pages over the groups if each `(slot, new tokens)` of
        `additions` were appended now (0: they all fit)."""
        worst = 0
        for g in self.groups:
            need = 0
            for slot, count in additions:
                start = self.lengths[slot]
                g.pages._check_length(start + count)
                release, take, _, _ = g.pages.plan(slot, start, start + count)
                need += len(take) - len(release)
            worst = max(worst, need - g.pages.allocator.num_free)
        return max(0, worst)

    def page_delta(self, slot: int, count: int) -> List[int]:
        """Pages each group would take, net of those it gives back, if `count` tokens were appended to `slot`."""
        start = self.lengths[slot]
        out = []
        for g in self.groups:
            g.pages._check_length(start + count)
            release, take, _, _ = g.pages.plan(slot, start, start + count)
            out.append(len(take) - len(release))
        return out

    def extend(self, additions: Sequence[Tuple[int, int]]) -> None:
        """Makes room for `count` more tokens of every `(slot, count)`: first gives back the
        pages that windows have passed, then takes new ones.  Raises OutOfPages, changing
        nothing, if a group lacks pages."""
        seen = set()
        for slot, count in additions:
            if not self.slots.is_held(slot):
                raise ValueError(f"slot {slot} is not in use")
            if slot in seen:
                raise ValueError(f"slot {slot} appears twice in one step")
            if count < 1:
                raise ValueError("a request brings at least one token to a step")
            seen.add(slot)
        short = self.pages_short(additions)
        if short > 0:
            raise OutOfPages(f"the step needs {short} more pages than the pool has free")
        for g in self.groups:
            plans = [(slot, g.pages.plan(slot, self.lengths[slot], self.lengths[slot] + count))
                     for slot, count in additions]
            for slot, (release, _, _, _) in plans:
                g.pages.give_back(slot, release)
            for slot, (_, take, new_lo, new_hi) in plans:
                g.pages.take(slot, take, new_lo, new_hi)
        for slot, count in additions:
            self.lengths[slot] += count

    def release(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise ValueError(f"slot {slot} is not in use")      # before any group is touched (a negative index would wrap)
        for g in self.groups:
            g.pages.release(slot)
        self.lengths[slot] = 0
        self.slots.free(slot)

    # ---- accounting --------------------------------------------------------
    def free_pages(self) -> int:
        return min((g.pages.allocator.num_free for g in self.groups), default=self.num_pages)

    def used_pages(self) -> int:
        return max((g.pages.allocator.num_used for g in self.groups), default=0)

    def worst_case_pages(self, total_tokens: int, largest_portion: int) -> int:
        return max((g.pages.worst_case_pages(total_tokens, largest_portion) for g in self.groups), default=0)

    def kv_bytes_per_token(self) -> int:
        """Bytes of keys and values one token adds over all cache entries."""
        size = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * len(g.cache_ids) * g.spec.num_kv_heads * g.spec.head_dim * size for g in self.groups)

    # ---- views for a step --------------------------------------------------
    def table_rows(self, group: int, slots: Sequence[int]) -> np.ndarray:
        return self.groups[group].pages.table[np.asarray(slots, dtype=np.int64)]

    def step_view(self, device_tables: Sequence[torch.Tensor]) -> "StepCacheView":
        return StepCacheView(self, device_tables)


class StepCacheView:
    """What the model sees of the cache during one step: per cache id the pools of its
    entry and the step's device copy of its group's block-table rows."""

    def __init__(self, manager: CacheManager, device_tables: Sequence[torch.Tensor]):
        self.manager = manager
        self.device_tables = device_tables

    def kv_view(self, cache_id: int, writes: bool) -> Optional[PagedKVView]:
        where = self.manager.entry_group.get(cache_id)
        if where is None:
            return None
        g, i = where
        group = self.manager.groups[g]
        return PagedKVView(spec=group.spec, k_pages=group.k_pool[i], v_pages=group.v_pool[i],
                           block_table=self.device_tables[g], page_size=self.manager.page_size, writes=writes)

    def state(self, cache_id: int) -> Optional[torch.Tensor]:
        return self.manager.states.get(cache_id)
