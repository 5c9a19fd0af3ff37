"""Page bookkeeping on the host: the free list and the per-request block tables of one group.

Grown from the reference's `BlockAllocator` (src/include/block_alloc.h:10-43: a LIFO
stack of page ids, first pops 0, 1, 2, ..., freed pages are taken again first) and the
table handling of `KVCacheManager` (src/include/kv_cache_manager.h:61-85).  Where the
reference returns -1 / false and lets the caller go on, this raises.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np


class OutOfPages(RuntimeError):
    """The pool has fewer free pages than a request needs."""


class PageAllocator:
    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise ValueError(f"a pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # pop() yields 0, 1, 2, ...
        self._held = np.zeros(num_pages, dtype=bool)

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        page = self._free.pop()
        self._held[page] = True
        return page

    def alloc_many(self, count: int) -> List[int]:
        """What `count` calls of `alloc` would hand out, in that order; nothing if the pool has fewer."""
        if count > len(self._free):
            raise OutOfPages(f"{count} pages needed, {len(self._free)} free")
        if count <= 0:
            return []
        pages = self._free[-count:]
        pages.reverse()
        del self._free[-count:]
        self._held[pages] = True
        return pages

    def free_many(self, pages: Sequence[int]) -> None:
        """`free` for each page in turn; nothing is freed if one of them is out of range, not held, or listed twice."""
        if len(pages) == 0:
            return
        ids = np.asarray(pages, dtype=np.int64)
        if ids.min() < 0 or ids.max() >= self.num_pages:
            raise ValueError(f"a page of {ids.tolist()} is outside the pool of {self.num_pages}")
        if not self._held[ids].all() or len(np.unique(ids)) != len(ids):
            raise ValueError(f"a page of {ids.tolist()} is freed twice (or was never handed out)")
        self._held[ids] = False
        self._free.extend(ids.tolist())

    def free(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise ValueError(f"page {page} is outside the pool of {self.num_pages}")
        if not self._held[page]:
            raise ValueError(f"page {page} is freed twice (or was never handed out)")
        self._held[page] = False
        self._free.append(page)

    def is_held(self, page: int) -> bool:
        return bool(self._held[page])


def pages_for(tokens: int, page_size: int) -> int:
    """ceil(tokens / page_size) (src/include/block_alloc.h:41-43)."""
    return (tokens + page_size - 1) // page_size


class GroupPages:
    """Pages and block tables of one cache group: layers whose keys and values have the
    same geometry and the same reach (all keys, or a window of them) share page ids."""

    def __init__(self, num_pages: int, page_size: int, max_slots: int, max_pages_per_request: int,
                 window: Optional[int] = None):
        self.page_size = page_size
        self.window = window
        self.allocator = PageAllocator(num_pages)
        self.max_pages_per_request = max_pages_per_request
        # table[slot, i]: physical page of the request's i-th logical page, -1 if none is held.
        self.table = np.full((max_slots, max_pages_per_request), -1, dtype=np.int32)
        # The request holds its logical pages lo..hi-1: table[slot, i] >= 0 exactly there.
        self._lo = [0] * max_slots                 # plain lists: read several times a step and request, as Python ints
        self._hi = [0] * max_slots

    # ---- what a range of new positions needs --------------------------------
    def first_needed_page(self, start: int) -> int:
        """First logical page that queries at positions >= start still read."""
        if self.window is None:
            return 0
        return max(0, start - self.window + 1) // self.page_size

    def plan(self, slot: int, start: int, end: int):
        """(logical pages to give back, logical pages to take, new lo, new hi) for running
        positions start..end-1 of `slot`."""
        lo, hi = self._lo[slot], self._hi[slot]
        need_lo, need_hi = self.first_needed_page(start), pages_for(end, self.page_size)
        release = range(lo, min(max(need_lo, lo), hi))
        take = range(max(hi, need_lo), need_hi)
        return release, take, max(lo, need_lo), max(hi, need_hi)

    def _check_length(self, end: int) -> None:
        if pages_for(end, self.page_size) > self.max_pages_per_request:
            raise OutOfPages(f"a request of {end} tokens needs {pages_for(end, self.page_size)} pages; "
                             f"its block table holds {self.max_pages_per_request}")

    def pages_short(self, slot: int, start: int, end: int) -> int:
        """How many pages the pool lacks for the range (0: it fits)."""
        self._check_length(end)
        release, take, _, _ = self.plan(slot, start, end)
        return max(0, len(take) - len(release) - self.allocator.num_free)

    def give_back(self, slot: int, logical_pages: range) -> None:
        if len(logical_pages):
            span = slice(logical_pages.start, logical_pages.stop)
            self.allocator.free_many(self.table[slot, span])
            self.table[slot, span] = -1

    def take(self, slot: int, logical_pages: range, new_lo: int, new_hi: int) -> None:
        if len(logical_pages):
            self.table[slot, logical_pages.start:logical_pages.stop] = self.allocator.alloc_many(len(logical_pages))
        self._lo[slot], self._hi[slot] = new_lo, new_hi

    def extend(self, slot: int, start: int, end: int) -> None:
        """Room for positions start..end-1 of one request: passed pages back, new pages in."""
        self._check_length(end)
        release, take, new_lo, new_hi = self.plan(slot, start, end)
        if len(take) - len(release) > self.allocator.num_free:
            raise OutOfPages(f"{len(take)} pages needed, {self.allocator.num_free + len(release)} available")
        self.give_back(slot, release)
        self.take(slot, take, new_lo, new_hi)

    def release(self, slot: int) -> None:
        lo, hi = self._lo[slot], self._hi[slot]
        self.allocator.free_many(self.table[slot, lo:hi])
        self.table[slot, lo:hi] = -1
        self._lo[slot] = self._hi[slot] = 0

    def held_pages(self, slot: int) -> List[int]:
        row = self.table[slot]
        return [int(p) for p in row[row >= 0]]

    def worst_case_pages(self, total_tokens: int, largest_portion: int) -> int:
        """Most pages a request of `total_tokens` holds at once when no step brings more
        than `largest_portion` of its tokens."""
        full = pages_for(total_tokens, self.page_size)
        if self.window is None:
            return full
        span = self.window - 1 + max(1, largest_portion)
        return min(full, pages_for(span, self.page_size) + 1)
