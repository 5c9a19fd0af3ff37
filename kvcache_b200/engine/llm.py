"""The Python entry point: token ids in, generated token ids out, through the scheduler, the
step function and the sampler.  It does in one process what the reference's driver does
around its binary (tools/run_serve.py:28-38: ids to the engine, generated ids back)."""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..config.options import EngineOptions
from ..sampling.params import SamplingParams
from .core import EngineCore
from .runner import StepEntry
from .scheduler import Request, Scheduler, TokensNeeded


class LLM:
    """`LLM(folder, dtype="bfloat16", ...).generate(prompts, params)` -> one id list per prompt."""

    def __init__(self, model: str, options: Optional[EngineOptions] = None, kernels=None, **option_fields):
        if options is None:
            options = EngineOptions(**option_fields)
        elif option_fields:
            raise ValueError("give either options or option fields, not both")
        if options.num_pages is None and options.max_cached_tokens is None:
            options.max_cached_tokens = 8192   # the reference's pool: 512 pages of 16 (apps/qwen_serve.cu:21)
        self.options = options
        self.core = EngineCore(model, options, kernels=kernels)
        self.config = self.core.config
        self.scheduler = self._new_scheduler()
        self._pending = None            # the step whose tokens have not been read yet
        self._step_events = []          # (begin, end) CUDA events of steps whose device time has not been read yet
        self._timing_events = []        # pairs that have been read: recorded again by later steps
        self.pipelined = True           # plan and launch a step before reading the one before it
        self.last_stats = None
        self.last_seconds = 0.0

    def _new_scheduler(self) -> Scheduler:
        o = self.options
        return Scheduler(self.core.cache, max_running=o.max_running, max_tokens_per_step=o.max_tokens_per_step,
                         chunk_size=o.chunk_size, max_model_len=self.core.max_model_len, admission=o.admission,
                         default_eos=getattr(self.config, "eos_token_ids", ()))

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._pending is not None

    def _launch(self, done: Optional[List[Request]] = None):
        """Plans and launches one step; returns (pieces, a function that waits for its tokens) or None.
        Requests that end because the pending step had to be read first are added to `done`."""
        try:
            pieces = self.scheduler.schedule()
        except TokensNeeded:
            finished = self._drain()          # pages are short: every token must be known before a request is preempted
            if done is not None:
                done += finished
            pieces = self.scheduler.schedule()
        if not pieces:
            return None
        entries = [StepEntry(p.request.slot, p.tokens, [p.count - 1] if p.samples else [],
                             (p.request.params.temperature, p.request.params.seed, p.output_index),
                             token_from_last=p.token_from_last)
                   for p in pieces]
        timed = self.core.device.type == "cuda"
        if timed:
            stream = self.core.runner.current_stream()
            begin, end = self._timing_events.pop() if self._timing_events else \
                (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            begin.record(stream)
        _, tokens = self.core.runner.step(entries, sample=True)
        if timed:
            end.record(stream)
            self._step_events.append((begin, end))
        self.scheduler.launched(pieces)
        count = sum(1 for p in pieces if p.samples)
        wait = self.core.runner.read_tokens_async(count) if count else (lambda: [])
        return pieces, wait

    def _must_wait_before_planning(self) -> bool:
        """Preemption recomputes a request from its tokens, so all of them must be known: with optimistic
        admission the pipeline is drained whenever pages are about to run short."""
        return (self.options.admission == "optimistic"
                and self.core.cache.free_pages() <= len(self.scheduler.running) + 1)

    def step(self) -> List[Request]:
        """One scheduler iteration.  The step is planned and launched before the previous step's tokens are
        read, so the host's work overlaps the device's; returns the requests that the tokens read in this
        call finished."""
        done: List[Request] = []
        if self._pending is not None and self._must_wait_before_planning():
            done += self._drain()
        launched = self._launch(done)
        done += self._drain()
        self._pending = launched
        if not self.pipelined:
            done += self._drain()
        return done

    def _drain(self) -> List[Request]:
        if self._pending is None:
            return []
        pieces, wait = self._pending
        self._pending = None
        tokens = wait()
        self._read_step_times()
        return self.scheduler.commit(pieces, tokens)

    def _read_step_times(self, wait: bool = False) -> None:
        """Adds the device time of the steps that have ended to the statistics (gpu_us of the reference's
        EngineStats, src/include/engine.h:37); never waits for a step unless `wait`."""
        while self._step_events:
            begin, end = self._step_events[0]
            if not end.query():
                if not wait:
                    return
                end.synchronize()
            self.scheduler.add_gpu_time(begin.elapsed_time(end) * 1e3)
            self._timing_events.append(self._step_events.pop(0))

    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[List[int]]:
        if params is None:
            params = SamplingParams()
        per_prompt = [params] * len(prompts) if isinstance(params, SamplingParams) else list(params)
        if len(per_prompt) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        self.scheduler = self._new_scheduler()
        self._pending = None
        self._step_events = []
        requests = [self.scheduler.add_request(p, sp) for p, sp in zip(prompts, per_prompt)]
        start = time.perf_counter()
        while self.has_work():
            before = self.scheduler.stats.steps
            self.step()
            if (self.scheduler.stats.steps == before and self._pending is None and self.scheduler.has_work()
                    and not self.scheduler.running):
                raise RuntimeError("the scheduler made no progress (a waiting request fits neither slots nor pages)")
        self.core.kernels.check_errors()
        self._read_step_times(wait=True)
        self.last_seconds = time.perf_counter() - start
        self.last_stats = self.scheduler.stats
        return [r.output for r in requests]
