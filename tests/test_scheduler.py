"""The scheduler's decisions, on the host alone: a fake step that only moves the cache's
bookkeeping and hands out tokens by rule."""
import numpy as np
import pytest

from kvcache_b200.cache import CacheManager
from kvcache_b200.engine.scheduler import FINISHED, RequestRejected, Scheduler
from kvcache_b200.parts.base import PagedKVSpec
from kvcache_b200.parts.model import CacheEntry
from kvcache_b200.sampling.params import SamplingParams


def _cache(num_pages=16, page=4, slots=4, window=None, max_tokens=256):
    return CacheManager([CacheEntry(PagedKVSpec(1, 8, window), None)], page_size=page, num_pages=num_pages,
                        max_slots=slots, max_tokens_per_request=max_tokens)


def _scheduler(cache, **kw):
    fields = dict(max_running=4, max_tokens_per_step=16, chunk_size=8, max_model_len=256, admission="reserve")
    fields.update(kw)
    return Scheduler(cache, **fields)


def _run_step(s: Scheduler, token=7):
    """What the engine does with a plan: extend the cache, then report one token per sampling piece."""
    pieces = s.schedule()
    if pieces:
        s.cache.extend([(p.request.slot, p.count) for p in pieces])
        for p in pieces:
            assert s.cache.length(p.request.slot) == p.start + p.count
        s.update(pieces, [token(p.request) if callable(token) else token for p in pieces if p.samples])
    return pieces


def _drain(s, token=7, limit=10_000):
    steps = []
    while s.has_work():
        pieces = _run_step(s, token)
        assert pieces, "the scheduler stalled"
        steps.append([(p.request.id, p.start, p.count, p.samples) for p in pieces])
        assert len(steps) < limit
    return steps


def test_portions_under_a_budget_then_decode():
    s = _scheduler(_cache())
    r = s.add_request(list(range(19)), SamplingParams(max_new_tokens=3, ignore_eos=True))
    steps = _drain(s)
    assert steps == [[(0, 0, 8, False)], [(0, 8, 8, False)], [(0, 16, 3, True)], [(0, 19, 1, True)], [(0, 20, 1, True)]]
    assert r.state == FINISHED and r.finish_reason == "length" and r.output == [7, 7, 7]
    assert s.cache.used_pages() == 0 and s.stats.generated == 3 and s.stats.finished == 1
    assert s.stats.prefill_tokens == 19 and s.stats.decode_tokens == 2


def test_max_new_one_gives_one_token():
    s = _scheduler(_cache())
    r = s.add_request([1, 2, 3], SamplingParams(max_new_tokens=1, ignore_eos=True))
    _drain(s)
    assert r.output == [7]


def test_decodes_go_first_and_prompts_share_what_is_left():
    s = _scheduler(_cache(num_pages=64), max_tokens_per_step=10, chunk_size=6)
    a = s.add_request([1] * 4, SamplingParams(max_new_tokens=5, ignore_eos=True))
    _run_step(s)                                   # a is prefetched whole and samples
    b = s.add_request([2] * 20, SamplingParams(max_new_tokens=2, ignore_eos=True))
    c = s.add_request([3] * 9, SamplingParams(max_new_tokens=2, ignore_eos=True))
    pieces = _run_step(s)
    assert [(p.request.id, p.count) for p in pieces] == [(0, 1), (1, 6), (2, 3)]     # 1 + 6 + 3 = budget
    pieces = _run_step(s)
    assert [(p.request.id, p.start, p.count) for p in pieces] == [(0, 5, 1), (1, 6, 6), (2, 3, 3)]
    assert all(len(step) <= 3 for step in _drain(s))
    assert [len(r.output) for r in (a, b, c)] == [5, 2, 2]


def test_eos_ends_and_is_kept_and_frees():
    s = _scheduler(_cache(), default_eos=(9,))
    r = s.add_request([1, 2], SamplingParams(max_new_tokens=10))
    q = s.add_request([1, 2], SamplingParams(max_new_tokens=4, ignore_eos=True))
    _drain(s, token=lambda req: 9 if len(req.output) == 2 else 5)
    assert r.output == [5, 5, 9] and r.finish_reason == "eos"
    assert q.output == [5, 5, 9, 5] and q.finish_reason == "length"


def test_reservation_blocks_in_arrival_order():
    """Worst case held back: 16 pages of 4; each request may need ceil((8 + 24) / 4) = 8 pages."""
    s = _scheduler(_cache(num_pages=16), max_tokens_per_step=64)
    reqs = [s.add_request([1] * 8, SamplingParams(max_new_tokens=24, ignore_eos=True)) for _ in range(3)]
    small = s.add_request([1], SamplingParams(max_new_tokens=1, ignore_eos=True))
    pieces = _run_step(s)
    assert [p.request.id for p in pieces] == [0, 1] and s.reserved == [16]
    assert reqs[2].state == "waiting" and small.state == "waiting"         # head-of-line: small waits behind 2
    steps = _drain(s)
    assert s.stats.preemptions == 0 and s.stats.peak_pages <= 16 and s.stats.peak_running == 2
    assert all(len(r.output) == 24 for r in reqs) and small.output == [7]
    assert s.reserved == [0]


def test_refused_at_submission():
    s = _scheduler(_cache(num_pages=4), max_model_len=64)
    with pytest.raises(RequestRejected, match="at least one"):
        s.add_request([], SamplingParams())
    with pytest.raises(RequestRejected, match="model length"):
        s.add_request([1] * 60, SamplingParams(max_new_tokens=5))
    with pytest.raises(RequestRejected, match="pages"):
        s.add_request([1] * 10, SamplingParams(max_new_tokens=8))          # 5 pages > pool of 4
    assert not s.has_work()


def test_optimistic_admission_preempts_the_newest_and_recomputes():
    s = _scheduler(_cache(num_pages=6, page=4), admission="optimistic", max_tokens_per_step=32, chunk_size=32)
    a = s.add_request([1] * 7, SamplingParams(max_new_tokens=12, ignore_eos=True))
    b = s.add_request([2] * 7, SamplingParams(max_new_tokens=12, ignore_eos=True))
    c = s.add_request([3] * 6, SamplingParams(max_new_tokens=3, ignore_eos=True))
    order = []
    counter = {"n": 0}

    def token(req):
        counter["n"] += 1
        return 100 + counter["n"]
    steps = _drain(s, token)
    assert s.stats.preemptions >= 1
    assert [len(r.output) for r in (a, b, c)] == [12, 12, 3]
    assert a.preemptions == 0                       # the oldest request is never the victim
    assert s.cache.used_pages() == 0
    # A preempted request runs its prompt and its earlier outputs again, from position 0.
    victim = b if b.preemptions else c
    restarts = [step for step in steps if any(i == victim.id and start == 0 for i, start, _, _ in step)]
    assert len(restarts) == victim.preemptions + 1


def test_optimistic_lone_request_that_cannot_grow_ends():
    s = _scheduler(_cache(num_pages=2, page=4, max_tokens=64), admission="optimistic", max_model_len=64)
    with pytest.raises(RequestRejected):
        s.add_request([1] * 6, SamplingParams(max_new_tokens=20, ignore_eos=True))
    # Two requests that each fit alone but not together: one is preempted, both finish.
    a = s.add_request([1] * 3, SamplingParams(max_new_tokens=5, ignore_eos=True))
    b = s.add_request([1] * 3, SamplingParams(max_new_tokens=5, ignore_eos=True))
    _drain(s)
    assert len(a.output) == 5 and len(b.output) == 5 and s.stats.preemptions >= 1


def test_window_requests_reserve_less():
    s = _scheduler(_cache(num_pages=8, page=4, window=8), chunk_size=4, max_tokens_per_step=8)
    # 100 tokens would need 25 pages with full attention; with a window of 8 at most ceil(11/4)+1 = 4.
    r = s.add_request([1] * 40, SamplingParams(max_new_tokens=60, ignore_eos=True))
    q = s.add_request([1] * 40, SamplingParams(max_new_tokens=60, ignore_eos=True))
    _drain(s)
    assert len(r.output) == 60 and len(q.output) == 60 and s.stats.peak_pages <= 8 and s.stats.peak_running == 2


def test_accounting_over_many_requests():
    """The reference's engine smoke test (apps/demo_engine.cu:13-44): totals and page bounds."""
    import random
    rng = random.Random(0)
    s = _scheduler(_cache(num_pages=64, page=4, slots=8), max_running=8, max_tokens_per_step=48, chunk_size=16)
    reqs = [s.add_request([1] * rng.randint(1, 40), SamplingParams(max_new_tokens=rng.randint(1, 30), ignore_eos=True))
            for _ in range(64)]
    _drain(s)
    assert s.stats.finished == 64 and s.stats.generated == sum(r.params.max_new_tokens for r in reqs)
    assert s.stats.peak_pages <= 64 and s.stats.peak_running <= 8 and s.cache.used_pages() == 0
    assert s.stats.prefill_tokens == sum(len(r.prompt) for r in reqs)


def test_pipelined_steps_with_late_tokens():
    """A step is planned while the tokens of the one before are still on their way: placeholders stand in,
    the next step takes the token from the device, an end token that arrives late drops the token computed
    after it, and a request at its length limit is not planned again."""
    s = _scheduler(_cache(), default_eos=(9,))
    a = s.add_request([1, 2, 3], SamplingParams(max_new_tokens=3))
    b = s.add_request([4, 5], SamplingParams(max_new_tokens=8))

    def launch():
        pieces = s.schedule()
        s.cache.extend([(p.request.slot, p.count) for p in pieces])
        s.launched(pieces)
        return pieces
    first = launch()
    assert [(p.request.id, p.count, p.samples, p.token_from_last) for p in first] == [(0, 3, True, -1), (1, 2, True, -1)]
    assert a.output == [-1] and b.output == [-1] and a.inflight == 1
    second = launch()                                   # planned before the first step's tokens are known
    assert [(p.request.id, p.start, p.count, p.token_from_last) for p in second] == [(0, 3, 1, 0), (1, 2, 1, 1)]
    assert second[0].tokens == [-1]
    s.commit(first, [5, 9])                             # b's first token is its end token
    assert a.output == [5, -1] and b.output == [9] and b.state == "finished" and b.finish_reason == "eos"
    third = launch()                                    # a's last token: afterwards it is not planned again
    assert [(p.request.id, p.token_from_last) for p in third] == [(0, 0)] and a.finishing
    assert s.commit(second, [6, 7]) == []               # 7 was computed for b after its end: dropped
    assert a.output == [5, 6, -1] and b.output == [9]
    assert launch() == []
    done = s.commit(third, [8])
    assert [r.id for r in done] == [0] and a.output == [5, 6, 8] and a.finish_reason == "length"
    assert not s.has_work() and s.cache.used_pages() == 0 and s.stats.generated == 4


def _pipelined(s, token=7, limit=10_000):
    """The entry point's loop on the host: a step is planned and launched before the tokens of the step before
    it are read; a plan that finds pages short while tokens are in flight has them read first."""
    from kvcache_b200.engine.scheduler import TokensNeeded
    pending = None
    steps = 0

    def read():
        nonlocal pending
        if pending is not None:
            pieces, pending = pending, None
            s.commit(pieces, [token(p.request) if callable(token) else token for p in pieces if p.samples])
    while s.has_work() or pending is not None:
        try:
            pieces = s.schedule()
        except TokensNeeded:
            read()
            pieces = s.schedule()
        if pieces:
            s.cache.extend([(p.request.slot, p.count) for p in pieces])
            s.launched(pieces)
        read()
        pending = pieces or None
        steps += 1
        assert steps < limit
        for r in list(s.running) + list(s.waiting):
            assert r.state != "waiting" or r.slot == -1
    return steps


@pytest.mark.parametrize("last_is_eos", [False, True])
def test_optimistic_preemption_waits_for_tokens_in_flight(last_is_eos):
    """20 pages of 4.  B brings a prompt of 70 tokens in portions of 32, A a prompt of 20.  When B's second portion
    lacks pages (8 + 5 held, 8 wanted), A's first token is still on its way - and it is A's last one (its length
    limit, or an end token).  A must not be preempted: it would be run again from a placeholder, and its end would
    free a slot it no longer holds.  The plan asks for the pending tokens instead; A ends and its pages serve B."""
    from kvcache_b200.engine.scheduler import TokensNeeded
    s = _scheduler(_cache(num_pages=20, page=4, max_tokens=128), admission="optimistic", max_tokens_per_step=64,
                   chunk_size=32, max_model_len=128, default_eos=(9,))
    b = s.add_request([2] * 70, SamplingParams(max_new_tokens=4, ignore_eos=True))
    a = s.add_request([1] * 20, SamplingParams(max_new_tokens=5) if last_is_eos else SamplingParams(max_new_tokens=1, ignore_eos=True))
    first = s.schedule()
    s.cache.extend([(p.request.slot, p.count) for p in first])
    s.launched(first)
    assert [(p.request.id, p.count, p.samples) for p in first] == [(0, 32, False), (1, 20, True)]
    assert s.cache.used_pages() == 13 and a.inflight == 1
    with pytest.raises(TokensNeeded):
        s.schedule()
    assert a.state == "running" and a.slot >= 0 and b.num_computed == 32 and s.stats.preemptions == 0
    done = s.commit(first, [9 if last_is_eos else 7])
    assert done == [a] and a.finish_reason == ("eos" if last_is_eos else "length") and a.output == [9 if last_is_eos else 7]
    _pipelined(s)
    assert b.output == [7] * 4 and s.cache.used_pages() == 0 and not s.running and not s.waiting
    assert s.stats.preemptions == 0


def test_optimistic_pipelined_generation_never_hands_out_a_placeholder():
    """Random loads under optimistic admission with tokens always one step late: every request ends with its
    full output, no placeholder, and every page comes back."""
    import random
    rng = random.Random(3)
    for trial in range(20):
        s = _scheduler(_cache(num_pages=12, page=4, slots=4, max_tokens=48), admission="optimistic", max_tokens_per_step=24,
                       chunk_size=rng.choice([4, 8, 16]), max_model_len=48)
        reqs = [s.add_request([1] * rng.randint(1, 20), SamplingParams(max_new_tokens=rng.randint(1, 12), ignore_eos=True))
                for _ in range(rng.randint(2, 8))]
        _pipelined(s)
        for r in reqs:
            assert r.state == "finished" and -1 not in r.output
            assert len(r.output) == r.params.max_new_tokens or r.finish_reason == "out_of_pages"
        assert s.cache.used_pages() == 0 and s.cache.slots.num_free == 4


def test_statistics_of_the_references_engine():
    """iters, tokens, slot and useful steps, latencies and wall time (src/include/engine.h:33-54), on a clock the
    test owns: every step takes one tick."""
    now = {"t": 0.0}
    s = _scheduler(_cache(num_pages=64), max_running=2, max_tokens_per_step=4, chunk_size=4, clock=lambda: now["t"])
    a = s.add_request([1] * 4, SamplingParams(max_new_tokens=2, ignore_eos=True))
    b = s.add_request([1] * 8, SamplingParams(max_new_tokens=1, ignore_eos=True))
    while s.has_work():
        pieces = s.schedule()
        s.cache.extend([(p.request.slot, p.count) for p in pieces])
        now["t"] += 1.0
        s.add_gpu_time(5.0)
        s.update(pieces, [7 for p in pieces if p.samples])
    # Steps: a's prompt (budget 4 leaves nothing for b, which is not yet admitted); a decodes + 3 tokens of b; b 3..7
    # (a has ended); b's last token + sampling.
    st = s.stats
    assert st.steps == 4 and st.generated == 3 and st.finished == 2 and st.gpu_us == 20.0
    assert a.finished_at == 2.0 and b.finished_at == 4.0
    assert st.avg_latency_us == pytest.approx(3.0e6) and st.p99_latency_us == pytest.approx(4.0e6) and st.wall_us == pytest.approx(4.0e6)
    assert st.slot_steps == 1 + 2 + 1 + 1 and st.useful_steps == 1 + 2 + 1 + 1 and st.slot_utilisation == 1.0


def test_a_piece_hands_out_its_tokens_without_joining_prompt_and_output():
    from kvcache_b200.engine.scheduler import Piece, Request
    request = Request(0, [5, 6, 7, 8], SamplingParams(max_new_tokens=4), output=[9, 10, 11])
    whole = request.tokens
    for start in range(len(whole)):
        for count in range(1, len(whole) - start + 1):
            assert list(Piece(request, start, count, False).tokens) == whole[start:start + count]
    inside = Piece(request, 1, 2, False).tokens
    assert isinstance(inside, np.ndarray) and inside.dtype == np.int32 and inside.base is request.prompt_ids
