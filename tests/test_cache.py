"""The cache manager's bookkeeping: pages, block tables, windows, slots.  No page is lost,
held twice or freed twice, under random orders of requests."""
import random

import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from kvcache_b200.cache import CacheManager, GroupPages, OutOfPages, OutOfSlots, PageAllocator, SlotAllocator, pages_for
from kvcache_b200.parts.base import PagedKVSpec, StateSpec
from kvcache_b200.parts.model import CacheEntry


def test_allocator_order_and_reuse():
    """First pops are 0, 1, 2, ...; freed pages are taken again first (src/include/block_alloc.h:14-32)."""
    a = PageAllocator(4)
    assert [a.alloc(), a.alloc()] == [0, 1]
    a.free(0)
    assert a.alloc() == 0 and a.alloc() == 2 and a.alloc() == 3
    with pytest.raises(OutOfPages):
        a.alloc()
    assert a.num_free == 0 and a.num_used == 4
    a.free(2)
    with pytest.raises(ValueError, match="twice"):
        a.free(2)
    with pytest.raises(ValueError):
        a.free(9)
    assert pages_for(17, 16) == 2 and pages_for(16, 16) == 1 and pages_for(0, 16) == 0


def test_many_pages_at_once_are_the_single_calls_in_turn():
    rng = random.Random(5)
    one, many = PageAllocator(40), PageAllocator(40)
    held = []
    for _ in range(200):
        if held and rng.random() < 0.45:
            k = rng.randint(1, min(6, len(held)))
            group = [held.pop(rng.randrange(len(held))) for _ in range(k)]
            for page in group:
                one.free(page)
            many.free_many(group)
        else:
            k = rng.randint(0, 7)
            if k > one.num_free:
                with pytest.raises(OutOfPages):
                    many.alloc_many(k)
                assert many.num_free == one.num_free
                continue
            singles = [one.alloc() for _ in range(k)]
            assert many.alloc_many(k) == singles
            held += singles
        assert one._free == many._free and (one._held == many._held).all()
    a = PageAllocator(6)
    pages = a.alloc_many(4)
    for bad in ([1, 1], [2, 5], [0, 6], [-1]):
        with pytest.raises(ValueError):
            a.free_many(bad)
        assert a.num_free == 2 and all(a.is_held(p) for p in pages)     # a refused call frees nothing
    a.free_many(np.asarray([3, 1], dtype=np.int32))
    assert a.alloc_many(2) == [1, 3]


def _manager(num_pages=8, page=4, slots=4, window=None, max_tokens=64, two_groups=False):
    entries = [CacheEntry(PagedKVSpec(2, 8, None), None), CacheEntry(PagedKVSpec(2, 8, None), None)]
    if window:
        entries += [CacheEntry(PagedKVSpec(2, 8, window), None)] if two_groups else []
        if not two_groups:
            entries = [CacheEntry(PagedKVSpec(2, 8, window), None)]
    return CacheManager(entries, page_size=page, num_pages=num_pages, max_slots=slots, max_tokens_per_request=max_tokens)


def test_reference_scenario():
    """The reference's unit test (tests/test_kv_manager.cu:11-59): 8 pages of 4 tokens."""
    m = _manager()
    assert len(m.groups) == 1 and m.groups[0].cache_ids == [0, 1]    # equal specs share a group
    a = m.admit()
    m.extend([(a, 5)])
    assert m.used_pages() == 2 and m.free_pages() == 6 and m.length(a) == 5
    for _ in range(3):
        m.extend([(a, 1)])
    assert m.used_pages() == 2 and m.length(a) == 8
    m.extend([(a, 1)])
    assert m.used_pages() == 3 and m.length(a) == 9
    b = m.admit()
    m.extend([(b, 20)])
    assert m.free_pages() == 0
    c = m.admit()
    assert m.pages_short([(c, 1)]) == 1
    with pytest.raises(OutOfPages):
        m.extend([(c, 1)])
    assert m.length(c) == 0 and m.groups[0].pages.held_pages(c) == []          # untouched
    with pytest.raises(OutOfPages):
        m.extend([(b, 1)])
    assert m.length(b) == 20
    m.release(a)
    assert m.free_pages() == 3
    m.extend([(b, 1)])
    assert m.length(b) == 21 and m.free_pages() == 2


def test_block_table_rows_and_reuse_order():
    m = _manager()
    a, b = m.admit(), m.admit()
    m.extend([(a, 6), (b, 3)])
    t = m.table_rows(0, [a, b])
    assert t[0, :2].tolist() == [0, 1] and t[1, 0] == 2 and (t[:, 3:] == -1).all()
    m.release(a)
    c = m.admit()
    m.extend([(c, 9)])
    assert m.table_rows(0, [c])[0, :3].tolist() == [1, 0, 3]      # a's pages first, last freed first


def test_step_is_atomic_over_entries():
    m = _manager(num_pages=4)
    a, b = m.admit(), m.admit()
    m.extend([(a, 4)])
    with pytest.raises(OutOfPages):
        m.extend([(a, 4), (b, 12)])        # 1 + 3 pages needed, 3 free
    assert m.length(a) == 4 and m.length(b) == 0 and m.used_pages() == 1
    with pytest.raises(ValueError, match="twice"):
        m.extend([(a, 1), (a, 1)])


def test_request_longer_than_its_table():
    m = _manager(max_tokens=16, num_pages=16)
    a = m.admit()
    with pytest.raises(OutOfPages, match="block table"):
        m.extend([(a, 17)])


def test_window_gives_pages_back():
    m = _manager(num_pages=6, page=4, window=6)
    a = m.admit()
    pages = m.groups[0].pages
    m.extend([(a, 10)])                          # positions 0..9: nothing can be dropped inside a step
    assert pages.held_pages(a) == [0, 1, 2]
    m.extend([(a, 1)])                           # query 10 sees keys 5..10: page 0 (0..3) goes back
    assert m.table_rows(0, [a])[0, :3].tolist() == [-1, 1, 2]
    for _ in range(40):                          # far beyond the pool's 24 tokens
        m.extend([(a, 1)])
    assert m.length(a) == 51 and len(pages.held_pages(a)) <= 3
    assert pages.first_needed_page(51) == (51 - 6 + 1) // 4
    m.release(a)
    assert m.free_pages() == 6


def test_groups_with_and_without_window_side_by_side():
    m = _manager(num_pages=8, page=4, window=6, two_groups=True)
    assert len(m.groups) == 2 and m.entry_group == {0: (0, 0), 1: (0, 1), 2: (1, 0)}
    a = m.admit()
    m.extend([(a, 20)])
    for _ in range(10):
        m.extend([(a, 1)])
    full, win = m.groups
    assert len(full.pages.held_pages(a)) == 8 and len(win.pages.held_pages(a)) <= 3
    assert m.pages_short([(a, 3)]) == 1           # the full group is the one that runs out
    assert m.worst_case_pages(100, 8) == 25 and win.pages.worst_case_pages(100, 8) == pages_for(6 - 1 + 8, 4) + 1


def test_slots():
    s = SlotAllocator(2)
    a, b = s.alloc(), s.alloc()
    assert (a, b) == (0, 1)
    with pytest.raises(OutOfSlots):
        s.alloc()
    s.free(a)
    with pytest.raises(ValueError):
        s.free(a)
    assert s.alloc() == 0


def test_state_slots_are_zeroed_at_admission():
    import torch
    entries = [CacheEntry(PagedKVSpec(1, 8, None), StateSpec((3, 2))), CacheEntry(None, StateSpec((5,), "float32"))]
    m = CacheManager(entries, page_size=4, num_pages=4, max_slots=3, max_tokens_per_request=16, dtype="float32", device="cpu")
    assert m.states[0].shape == (3, 3, 2) and m.states[1].shape == (3, 5) and m.entry_group == {0: (0, 0)}
    a = m.admit()
    m.states[1][a] += 7
    m.release(a)
    assert m.admit() == a and float(m.states[1][a].abs().sum()) == 0.0
    assert m.groups[0].k_pool.shape == (1, 4, 1, 4, 8)


def _check_invariants(m: CacheManager, live):
    for g in m.groups:
        held = [p for slot in live for p in g.pages.held_pages(slot)]
        assert len(held) == len(set(held)), "a page is held twice"
        assert len(held) == g.pages.allocator.num_used, "a page is lost"
        assert sorted(held + g.pages.allocator._free) == list(range(m.num_pages)), "free list and tables disagree"
        for slot in live:
            n = m.length(slot)
            first = g.pages.first_needed_page(n - 1) if n else 0
            row = g.pages.table[slot]
            for i in range(first, pages_for(n, m.page_size)):
                assert row[i] >= 0, "a page that is still read was given back"


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 2 ** 32 - 1), st.sampled_from([None, 5, 16]), st.sampled_from([2, 4, 8]))
def test_random_orders_keep_the_books(seed, window, page):
    rng = random.Random(seed)
    m = _manager(num_pages=12, page=page, slots=4, window=window, max_tokens=200, two_groups=window is not None)
    live = []
    for _ in range(120):
        action = rng.random()
        if action < 0.25 and len(live) < 4:
            live.append(m.admit())
        elif action < 0.4 and live:
            m.release(live.pop(rng.randrange(len(live))))
        elif live:
            chosen = rng.sample(live, rng.randint(1, len(live)))
            additions = [(s, rng.choice([1, 1, 1, 2, 7, 13])) for s in chosen]
            before = [m.length(s) for s in live]
            try:
                m.extend(additions)
            except OutOfPages:
                assert [m.length(s) for s in live] == before
        _check_invariants(m, live)
    for s in live:
        m.release(s)
    assert m.used_pages() == 0 and m.slots.num_free == 4
