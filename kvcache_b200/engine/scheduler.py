"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.  Host logic only; it talks to the cache manager's bookkeeping and never
to the device.

Grown from the reference's loop (apps/qwen_serve.cu:177-204) and toy engine
(src/include/engine.h:100-140): retire, then admit in arrival order while the batch has room
and the worst case of every admitted request still fits the pool
(`reserved + ceil((prompt + max_new) / page) <= pages`, engine.h:114-124), then one decode
token for every running request.  What is new here: a step mixes decode tokens with portions
of prompts (the reference prefills each prompt whole and alone, qwen_serve.cu:90-124); a
request is checked for its end right after sampling, so `max_new = 1` yields one token (the
reference yields two, qwen_serve.cu:192-203); and a request that can never fit is refused
when it is submitted (the reference's loop would spin forever, qwen_serve.cu:195,201).

Pipelining.  A step's sampled tokens need not be known on the host before the next step is
planned: `launched(pieces)` records that a step is on its way (its sampling requests get a
placeholder token, which the next step reads on the device), `commit(pieces, tokens)` fills the
placeholders in when the tokens arrive and ends requests.  A request whose end token arrives
after it was already given a place in the following step simply has that step's token dropped.
`update` is the two in one, for callers that wait for every step.

When pages run out.  `admission="reserve"` (default): they cannot, because every admitted
request's worst case is held back.  `admission="optimistic"`: a request is admitted when its
next portion fits; if a later step lacks pages, the newest running request is preempted - its
pages and slot are given back, it returns to the head of the waiting queue and its tokens are
run again later - until the step fits.  A lone request that cannot grow any further ends with
reason "out_of_pages".
"""
from __future__ import annotations

import bisect
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

import numpy as np

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


class RequestRejected(ValueError):
    pass


class TokensNeeded(RuntimeError):
    """`schedule()` found pages short while a step's tokens are still on their way.  Preempting recomputes a request
    from its tokens and ending one hands its output out, so both need every token known: read the pending step
    (`commit`) and call `schedule()` again.  Nothing was changed."""


@dataclass
class Request:
    id: int
    prompt: List[int]
    params: SamplingParams
    eos: Tuple[int, ...] = ()
    state: str = WAITING
    slot: int = -1
    output: List[int] = field(default_factory=list)
    num_computed: int = 0          # tokens of prompt + output already run through the model
    finish_reason: Optional[str] = None
    preemptions: int = 0
    reserved: Optional[List[int]] = None   # pages held back for it in each group (reserve policy)
    inflight: int = 0              # placeholders at the end of `output`: sampled, not yet known on the host
    last_index: int = -1           # where the step that sampled the newest placeholder put it (device order)
    finishing: bool = False        # its last token is on its way: it takes no part in further steps
    arrival: float = 0.0           # seconds on the scheduler's clock when it was submitted
    finished_at: Optional[float] = None
    prompt_ids: Optional[np.ndarray] = None   # the prompt as int32, made once: a portion of it is a view, not a copy

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    def span(self, start: int, count: int):
        """Tokens start..start+count-1 of prompt + output, without joining the two."""
        n, end = len(self.prompt), start + count
        if end <= n:
            if self.prompt_ids is None:
                self.prompt_ids = np.asarray(self.prompt, dtype=np.int32)
            return self.prompt_ids[start:end]
        if start >= n:
            return self.output[start - n:end - n]
        return self.prompt[start:] + self.output[:end - n]

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)


PLACEHOLDER = -1


@dataclass
class Piece:
    """One request's share of a step."""
    request: Request
    start: int                     # first position run in this step
    count: int
    samples: bool                  # the piece ends at the request's last token: a token is sampled
    output_index: int = -1         # which element of request.output the sampled token becomes
    token_from_last: int = -1      # >= 0: its (single) token is the previous step's sampled token at this index

    @property
    def tokens(self) -> Sequence[int]:
        return self.request.span(self.start, self.count)


@dataclass
class SchedulerStats:
    """The reference's EngineStats (src/include/engine.h:33-45: iters, tokens, gpu_us, wall_us, slot_steps,
    useful_steps, peak_blocks, finished, avg and p99 latency) plus portion counts and preemptions."""
    steps: int = 0                 # iters
    decode_tokens: int = 0
    prefill_tokens: int = 0
    generated: int = 0             # tokens
    finished: int = 0
    preemptions: int = 0
    peak_running: int = 0
    peak_pages: int = 0            # peak_blocks
    gpu_us: float = 0.0            # device time of the steps, where the caller measures it (`add_gpu_time`)
    wall_us: float = 0.0           # first submission to last end, on the scheduler's clock
    slot_steps: int = 0            # sum over steps of the requests that held a slot
    useful_steps: int = 0          # sum over steps of the requests that had tokens in the step
    avg_latency_us: float = 0.0    # submission to end, over finished requests
    p99_latency_us: float = 0.0

    @property
    def slot_utilisation(self) -> float:
        return self.useful_steps / self.slot_steps if self.slot_steps else 0.0


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_running: int, max_tokens_per_step: int, chunk_size: int,
                 max_model_len: int, admission: str = "reserve", default_eos: Sequence[int] = (),
                 clock=time.perf_counter):
        if admission not in ("reserve", "optimistic"):
            raise ValueError(f"unknown admission policy '{admission}'")
        self.cache = cache
        self.max_running = min(max_running, cache.max_slots)
        self.max_tokens_per_step = max_tokens_per_step
        self.chunk_size = chunk_size
        self.max_model_len = max_model_len
        self.admission = admission
        self.default_eos = tuple(default_eos)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: List[Request] = []
        self.reserved = [0] * len(cache.groups)
        self.stats = SchedulerStats()
        self._next_id = 0
        self._clock = clock
        self._first_arrival: Optional[float] = None
        self._latencies: List[float] = []

    # ---- submission --------------------------------------------------------
    def _worst_case(self, total_tokens: int) -> List[int]:
        return [g.pages.worst_case_pages(total_tokens, self.chunk_size) for g in self.cache.groups]

    def add_request(self, prompt: Sequence[int], params: SamplingParams) -> Request:
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise RequestRejected("a request needs at least one prompt token")
        total = len(prompt) + params.max_new_tokens
        if total > self.max_model_len:
            raise RequestRejected(f"prompt ({len(prompt)}) + max_new_tokens ({params.max_new_tokens}) exceeds the "
                                  f"model length {self.max_model_len}")
        worst = self._worst_case(total)
        if any(w > self.cache.num_pages for w in worst):
            raise RequestRejected(f"the request can need {max(worst)} pages; the pool has {self.cache.num_pages}")
        eos = () if params.ignore_eos else (params.eos_token_ids if params.eos_token_ids is not None else self.default_eos)
        request = Request(self._next_id, prompt, params, eos=tuple(eos), arrival=self._clock())
        if self._first_arrival is None:
            self._first_arrival = request.arrival
        self._next_id += 1
        self.waiting.append(request)
        return request

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- one step's plan ---------------------------------------------------
    def _admit(self, request: Request) -> None:
        request.slot = self.cache.admit()
        request.state = RUNNING
        if self.admission == "reserve":
            request.reserved = self._worst_case(len(request.prompt) + request.params.max_new_tokens)
            for g, pages in enumerate(request.reserved):
                self.reserved[g] += pages
        self.running.append(request)

    def _can_reserve(self, request: Request) -> bool:
        worst = self._worst_case(len(request.prompt) + request.params.max_new_tokens)
        return all(self.reserved[g] + w <= self.cache.num_pages for g, w in enumerate(worst))

    def _retire(self, request: Request, reason: str) -> None:
        request.state, request.finish_reason = FINISHED, reason
        self._give_back(request)
        self.running.remove(request)
        self.finished.append(request)
        stats = self.stats
        stats.finished += 1
        # Latency figures as the reference fills them (src/include/engine.h:47-54): mean, and the sample at 0.99 n.
        request.finished_at = self._clock()
        bisect.insort(self._latencies, (request.finished_at - request.arrival) * 1e6)
        ordered = self._latencies
        stats.avg_latency_us = sum(ordered) / len(ordered)
        stats.p99_latency_us = ordered[min(int(len(ordered) * 0.99), len(ordered) - 1)]
        stats.wall_us = (request.finished_at - self._first_arrival) * 1e6

    def add_gpu_time(self, microseconds: float) -> None:
        """Device time of a step, measured by the caller (the scheduler itself never touches the device)."""
        self.stats.gpu_us += microseconds

    def _give_back(self, request: Request) -> None:
        if request.slot < 0:
            raise AssertionError(f"request {request.id} holds no slot")
        self.cache.release(request.slot)
        request.slot = -1
        if request.reserved is not None:
            for g, pages in enumerate(request.reserved):
                self.reserved[g] -= pages
            request.reserved = None

    def _preempt_newest(self, keep: Optional[Request] = None) -> Optional[Request]:
        """Gives back the newest running request's pages; it waits again, first in line."""
        for victim in reversed(self.running):
            if victim is keep or victim.inflight or victim.finishing:
                continue                      # its tokens are not all known, or it ends with the token on its way
            self._give_back(victim)
            self.running.remove(victim)
            victim.state, victim.num_computed = WAITING, 0
            victim.preemptions += 1
            self.stats.preemptions += 1
            self.waiting.appendleft(victim)
            return victim
        return None

    def schedule(self) -> List[Piece]:
        """Chooses this step's pieces: one token for every running request that is decoding,
        then portions of unfinished prompts (oldest first), then newly admitted requests, all
        under the token budget and the pages that are free.  May preempt (optimistic policy)."""
        budget = self.max_tokens_per_step
        pieces: List[Piece] = []
        groups = self.cache.groups
        need = [0] * len(groups)          # pages the pieces placed so far take, net of what they give back

        def delta(request: Request, count: int) -> List[int]:
            return self.cache.page_delta(request.slot, count)

        def fits(request: Request, count: int) -> bool:
            d = delta(request, count)
            return all(need[g] + d[g] <= groups[g].pages.allocator.num_free for g in range(len(groups)))

        def place(request: Request, count: int) -> None:
            nonlocal budget
            start = request.num_computed
            d = delta(request, count)
            for g in range(len(groups)):
                need[g] += d[g]
            from_last = request.last_index if (request.inflight and count == 1 and start == request.num_tokens - 1) else -1
            pieces.append(Piece(request, start, count, start + count == request.num_tokens,
                                output_index=len(request.output), token_from_last=from_last))
            budget -= count

        def recount() -> None:
            nonlocal budget
            for g in range(len(groups)):
                need[g] = 0
            for p in pieces:
                d = delta(p.request, p.count)
                for g in range(len(groups)):
                    need[g] += d[g]
            budget = self.max_tokens_per_step - sum(p.count for p in pieces)

        # Running requests, oldest first: decodes take one token, prompts a portion.
        index = 0
        while index < len(self.running):
            request = self.running[index]
            remaining = request.num_tokens - request.num_computed
            count = min(remaining, self.chunk_size, budget)
            if count <= 0 or request.finishing:
                index += 1
                continue
            if not fits(request, count) and self.has_inflight():
                # Nothing has been changed yet: tokens in flight stay in flight during a plan, so no earlier
                # request of this loop can have preempted or ended anything.
                raise TokensNeeded("pages are short and a step's tokens have not been read yet")
            while not fits(request, count):
                victim = self._preempt_newest(keep=request)
                if victim is None:
                    break
                # Drop what the victim had been given in this step.
                pieces[:] = [p for p in pieces if p.request is not victim]
                recount()
            if not fits(request, count):
                smaller = count
                while smaller > 1 and not fits(request, smaller):
                    smaller -= 1
                if fits(request, smaller) and smaller < remaining:
                    count = smaller           # a shorter portion of a prompt still makes progress
                else:
                    self._retire(request, "out_of_pages")
                    continue
            place(request, count)
            index += 1

        # Waiting requests, in arrival order; the first that does not fit blocks the rest.
        while self.waiting and len(self.running) < self.max_running and budget > 0:
            request = self.waiting[0]
            if self.admission == "reserve" and not self._can_reserve(request):
                break
            count = min(request.num_tokens - request.num_computed, self.chunk_size, budget)
            self.waiting.popleft()
            self._admit(request)
            if not fits(request, count):
                # Not even its first portion fits now: back to the head of the queue.
                self._give_back(request)
                self.running.remove(request)
                request.state = WAITING
                self.waiting.appendleft(request)
                break
            place(request, count)

        self.stats.peak_running = max(self.stats.peak_running, len(self.running))
        return pieces

    # ---- after the step ----------------------------------------------------
    def launched(self, pieces: Sequence[Piece]) -> None:
        """The step is on its way to the device: positions advance, sampling requests get a placeholder
        for the token to come, and a request whose last token this is takes no part in later steps."""
        self.stats.steps += 1
        self.stats.slot_steps += len(self.running)
        self.stats.useful_steps += len(pieces)
        k = 0
        for piece in pieces:
            request = piece.request
            request.num_computed += piece.count
            if piece.count == 1 and piece.start >= len(request.prompt):
                self.stats.decode_tokens += 1
            else:
                self.stats.prefill_tokens += piece.count
            if not piece.samples:
                continue
            piece.output_index = len(request.output)
            request.output.append(PLACEHOLDER)
            request.inflight += 1
            request.last_index = k
            k += 1
            if len(request.output) >= request.params.max_new_tokens or request.num_tokens >= self.max_model_len:
                request.finishing = True
        self.stats.peak_pages = max(self.stats.peak_pages, self.cache.used_pages())

    def commit(self, pieces: Sequence[Piece], sampled: Sequence[int]) -> List[Request]:
        """The step's tokens have arrived: `sampled` holds one for every piece with `samples`, in order.
        Returns the requests that finished."""
        done: List[Request] = []
        it = iter(sampled)
        for piece in pieces:
            if not piece.samples:
                continue
            token = int(next(it))
            request = piece.request
            if request.state == FINISHED or piece.output_index >= len(request.output):
                continue                      # it ended on an earlier token; this one was computed in vain
            request.output[piece.output_index] = token
            request.inflight -= 1
            self.stats.generated += 1
            if token in request.eos:
                reason = "eos"
                del request.output[piece.output_index + 1:]      # a placeholder of the step that followed
            elif piece.output_index + 1 >= request.params.max_new_tokens:
                reason = "length"
            elif len(request.prompt) + piece.output_index + 1 >= self.max_model_len:
                reason = "model_length"
            else:
                continue
            request.inflight = 0
            self._retire(request, reason)
            done.append(request)
        return done

    def has_inflight(self) -> bool:
        return any(r.inflight for r in self.running)

    def update(self, pieces: Sequence[Piece], sampled: Sequence[int]) -> List[Request]:
        """`launched` and `commit` in one, for a caller that waits for every step's tokens."""
        self.launched(pieces)
        return self.commit(pieces, sampled)
