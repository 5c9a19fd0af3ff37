"""Benchmark of kvcache_b200: decode tokens a second of the Qwen2.5-0.5B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on standard output.  `value`: decoded tokens a second at batch 8 and the
benchmark context (device-timed decode steps through the engine's step function and device
sampler); `e2e`: the same through the Python entry point (`LLM.step`: host token ids in,
host token ids out, scheduler and copies included); `prefill`: one 2,048-token prompt;
`roofline`: bytes a decode step has to read (every weight once, the cache of the live
requests) over its time, against the measured copy bandwidth, and the same for each class
of kernel of the step (`roofline.kernels`, CUDA events around every launch of a step that
is launched kernel by kernel); `points`: decode at batch 1 and 64, and the reference's own
published workload (one request, a prompt of 29 tokens, 256 new tokens, wall clock per
token: README.md:143-148 of kimxinw/kvcache).  Weights are seeded random numbers of the
named shape, prompts are random ids, and the cache of the timed requests is filled with
random keys and values instead of being prefilled (`data`: synthetic).

`--impl reference` runs kimxinw/kvcache itself, unmodified, compiled for sm_100a under
`baseline/_ref` (see baseline/reference_arm.py): the same eight requests at the same
context through its `qwen_serve`, whose pool of 512 pages of 16 tokens admits two such
requests at a time (apps/qwen_serve.cu:21,192-200), and one request through its
`qwen_infer` with CUDA-graph decode for the batch-1 points.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Qwen2.5-0.5B layer sizes (the third configuration the baseline names).
QWEN25_05B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 896, "num_hidden_layers": 24,
    "num_attention_heads": 14, "num_key_value_heads": 2, "intermediate_size": 4864, "vocab_size": 151936,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": True, "max_position_embeddings": 32768,
    "hidden_act": "silu", "use_sliding_window": False, "sliding_window": 32768, "max_window_layers": 24,
    "eos_token_id": 151645,
}
CONTEXT = 4096
PREFILL_TOKENS = 2048
# The reference's best published decode: 8,104 us a token - one request, a prompt of 29 tokens, 256 new tokens,
# CUDA-graph decode, float16, on an RTX 3060 (README.md:143-148 of kimxinw/kvcache).
PUBLISHED_TOK_S = 1e6 / 8104.0
PUBLISHED_PROMPT, PUBLISHED_NEW = 29, 256
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
REFERENCE_MAX_STEPS = 64            # the reference decodes a token in about 0.12 s at this context


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as fh:
            data = json.load(fh)
        return {"hbm_gbs": float(data.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"])),
                "bf16_tflops": float(data.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"])),
                "bf16_tflops_sustained": float(data.get("bf16_tflops_sustained", data.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))),
                "source": "measured"}
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """SM clock and slowdown reasons of GPU 0, read every two milliseconds for the whole run (NVML in this process;
    `nvidia-smi -lms` where the NVML binding is missing).  Every timed region is bracketed with `region(name)`; its
    record holds the samples that fell inside it.  Reading only: no setting of the GPU is touched."""
    REASONS = (("hw_slowdown", "nvmlClocksEventReasonHwSlowdown"), ("hw_thermal_slowdown", "nvmlClocksEventReasonHwThermalSlowdown"),
               ("sw_thermal_slowdown", "nvmlClocksEventReasonSwThermalSlowdown"), ("sw_power_cap", "nvmlClocksEventReasonSwPowerCap"))

    def __init__(self, interval: float = 0.002):
        self.interval = interval
        self.samples = []            # (time, sm MHz, set of reasons)
        self.max_mhz = None
        self.regions = {}
        self.how = None
        self._stop = threading.Event()
        self._thread = None
        self._proc = None

    def start(self, wait: float = 3.0) -> "ClockSampler":
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(0).uuid)
            try:
                handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid if not uuid.startswith("GPU-") else uuid).encode())
            except Exception:
                handle = pynvml.nvmlDeviceGetHandleByIndex(0)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            masks = [(name, getattr(pynvml, attr)) for name, attr in self.REASONS]

            def poll():
                while not self._stop.is_set():
                    try:
                        mhz = int(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
                        word = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                        self.samples.append((time.perf_counter(), mhz, frozenset(n for n, m in masks if word & m)))
                    except Exception:
                        pass
                    self._stop.wait(self.interval)
            self.how = "nvml"
            self._thread = threading.Thread(target=poll, daemon=True)
            self._thread.start()
        except Exception:
            self._start_smi()
        deadline = time.perf_counter() + wait
        while not self.samples and time.perf_counter() < deadline:
            time.sleep(0.01)
        return self

    def _start_smi(self):
        query = "clocks.sm,clocks.max.sm," + ",".join(f"clocks_event_reasons.{name}" for name, _ in self.REASONS)
        try:
            self._proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={query}", "--format=csv,noheader,nounits",
                                           "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.how = "unavailable"
            return
        self.how = "nvidia-smi"

        def read():
            for line in self._proc.stdout:
                fields = [f.strip() for f in line.split(",")]
                try:
                    mhz, self.max_mhz = int(fields[0]), int(fields[1])
                except (ValueError, IndexError):
                    continue
                active = frozenset(name for (name, _), v in zip(self.REASONS, fields[2:6]) if v.lower().startswith("active"))
                self.samples.append((time.perf_counter(), mhz, active))
        self._thread = threading.Thread(target=read, daemon=True)
        self._thread.start()

    @contextlib.contextmanager
    def region(self, name: str):
        begin = time.perf_counter()
        try:
            yield
        finally:
            self.regions[name] = self._summary(begin, time.perf_counter())

    def _summary(self, begin: float, end: float):
        inside = [(mhz, reasons) for t, mhz, reasons in list(self.samples) if begin <= t <= end]
        reasons = sorted(set().union(*[r for _, r in inside])) if inside else []
        return {"sm_mhz": statistics.median(m for m, _ in inside) if inside else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(inside)}

    def stop(self):
        self._stop.set()
        if self._proc is not None:
            self._proc.terminate()


def make_folder(tmp: str, layers: int) -> str:
    import torch
    import kvcache_b200  # noqa: F401
    from kvcache_b200.config import config_from_dict
    from kvcache_b200.weights import write_random_model
    config = dict(QWEN25_05B, num_hidden_layers=layers, max_window_layers=layers)
    return write_random_model(os.path.join(tmp, "qwen25_05b_random"), config_from_dict(config), seed=0, dtype=torch.bfloat16)


def bench_config(batch: int, layers: int, steps: int, warmup: int, peaks_source: str) -> dict:
    """What both arms run: the named model, eight requests, each with about CONTEXT tokens cached while its
    `steps` timed tokens are decoded (after `warmup` untimed ones)."""
    c = QWEN25_05B
    return {"model": "Qwen2.5-0.5B shape, random weights", "global_batch": batch, "seq_len": CONTEXT,
            "parallelism": "single GPU", "layers": layers, "layers_of_model": c["num_hidden_layers"],
            "hidden": c["hidden_size"], "q_heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"],
            "head_dim": c["hidden_size"] // c["num_attention_heads"], "intermediate": c["intermediate_size"],
            "vocab": c["vocab_size"], "page_size": 16, "new_tokens": steps + warmup,
            "prefill_tokens": PREFILL_TOKENS, "l2": "inputs larger than L2 (weights read once per step)",
            "peaks": peaks_source, "published_hw": "RTX 3060 (vs_baseline divides by its batch-1 number)"}


METRIC = "decode tok/s at batch 8 (Qwen2.5-0.5B shape, context 4096)"


def fill_cache_randomly(core, slots, context):
    """Gives each slot `context` cached tokens of random keys and values (no prefill run)."""
    import torch
    core.cache.extend([(s, context) for s in slots])
    g = torch.Generator(device=core.device).manual_seed(1)
    for group in core.cache.groups:
        group.k_pool.normal_(0.0, 1.0, generator=g)
        group.v_pool.normal_(0.0, 1.0, generator=g)


def _decode_engine(folder, batch, context, use_graphs=True):
    from kvcache_b200.config.options import EngineOptions
    from kvcache_b200.engine.core import EngineCore
    options = EngineOptions(dtype="bfloat16", page_size=16, max_cached_tokens=batch * (context + 16), max_running=batch,
                            max_tokens_per_step=max(batch, 16), max_model_len=context + 16, use_graphs=use_graphs)
    return EngineCore(folder, options)


def time_decode(folder, batch, context, steps, warmup, clocks, name, use_graphs=True):
    """Device-timed decode steps at `batch` requests of about `context` cached tokens each."""
    import torch
    from kvcache_b200.engine.decode_loop import DecodeLoop
    core = _decode_engine(folder, batch, context, use_graphs)
    slots = [core.cache.admit() for _ in range(batch)]
    start_len = context - steps - warmup
    fill_cache_randomly(core, slots, start_len)
    loop = DecodeLoop(core, slots, use_graphs=use_graphs)
    tokens = torch.randint(0, core.model.vocab_size, (batch,), generator=torch.Generator().manual_seed(2), dtype=torch.int32)
    loop.set_tokens(tokens)
    for _ in range(warmup):
        loop.step()
    torch.cuda.synchronize()
    launches_before = loop.launches
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    with clocks.region(name):
        marks[0].record()
        for i in range(steps):
            loop.step()
            marks[i + 1].record()
        torch.cuda.synchronize()
    core.kernels.check_errors()
    ms = marks[0].elapsed_time(marks[-1])
    per_step = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
    mean_context = start_len + warmup + (steps - 1) / 2.0 + 1
    step_bytes = core.model.decode_weight_bytes() + batch * mean_context * core.cache.kv_bytes_per_token()
    result = {"ms_per_step": ms / steps, "ms_p50": per_step[len(per_step) // 2], "tok_s": batch * steps / (ms / 1e3),
              "bytes_per_step": step_bytes, "launches": loop.launches - launches_before}
    del loop, core
    torch.cuda.empty_cache()
    return result


def time_kernel_classes(folder, batch, context, peaks, repeats=5):
    """One decode step launched kernel by kernel with CUDA events around every launch: microseconds, bytes the class
    has to move and the fraction of the measured copy bandwidth, for each class of kernel.  A kernel timed alone waits
    for the one before it and cannot start early, so the classes add up to more than a replayed step takes."""
    import torch
    from kvcache_b200.engine.decode_loop import DecodeLoop
    core = _decode_engine(folder, batch, context, use_graphs=False)
    timing = getattr(core.kernels, "start_timing", None)
    if timing is None:
        return None
    slots = [core.cache.admit() for _ in range(batch)]
    fill_cache_randomly(core, slots, context - repeats - 4)
    loop = DecodeLoop(core, slots, use_graphs=False)
    loop.set_tokens(torch.zeros(batch, dtype=torch.int32))
    for _ in range(3):
        loop.step()
    torch.cuda.synchronize()
    core.kernels.start_timing(hold_ms=12.0)           # longer than the host needs to queue a step's launches and events
    for _ in range(repeats):
        loop.step()
    report = core.kernels.stop_timing()
    out = {}
    for name, entry in report.items():
        us = entry["us"] / repeats
        item = {"us": round(us, 2), "launches": entry["launches"] // repeats}
        if entry["bytes"]:
            gbs = entry["bytes"] / repeats / (us * 1e-6) / 1e9
            item.update({"mb": round(entry["bytes"] / repeats / 1e6, 2), "gbs": round(gbs, 1), "frac": round(gbs / peaks["hbm_gbs"], 3)})
        out[name] = item
    del loop, core
    torch.cuda.empty_cache()
    return out


def time_prefill(folder, tokens, clocks, repeats=3, warm=5):
    import torch
    from kvcache_b200.config.options import EngineOptions
    from kvcache_b200.engine.core import EngineCore
    from kvcache_b200.engine.runner import StepEntry
    options = EngineOptions(dtype="bfloat16", page_size=16, max_cached_tokens=tokens + 16, max_running=1,
                            max_tokens_per_step=tokens, max_model_len=tokens + 16, use_graphs=True)
    core = EngineCore(folder, options)
    ids = torch.randint(0, core.model.vocab_size, (tokens,), generator=torch.Generator().manual_seed(3)).to(torch.int32).numpy()
    times = []                                       # host token ids, as the scheduler hands a prompt's portion to the step
    with clocks.region("prefill"):
        for i in range(warm + repeats):              # the step is replayed from a graph once its shape has come a few times
            slot = core.cache.admit()
            torch.cuda.synchronize()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            core.runner.step([StepEntry(slot, ids, [tokens - 1])])
            end.record()
            torch.cuda.synchronize()
            core.cache.release(slot)
            if i >= warm:
                times.append(begin.elapsed_time(end))
    core.kernels.check_errors()
    c = core.config
    per_layer = 2 * tokens * c.hidden_size * (c.q_size + 2 * c.kv_size) + 2 * tokens * c.q_size * c.hidden_size \
        + 3 * 2 * tokens * c.hidden_size * c.intermediate_size + 4 * c.num_attention_heads * c.head_dim * tokens * (tokens + 1) / 2
    flops = c.num_hidden_layers * per_layer + 2 * c.hidden_size * c.vocab_size
    ms = statistics.median(times)
    del core
    torch.cuda.empty_cache()
    return {"ms": ms, "tok_s": tokens / (ms / 1e3), "flops": flops}


def time_e2e(folder, batch, context, steps, warmup, clocks):
    """Decode through the Python entry point: every step the scheduler plans, the step's token ids
    go from pinned host memory to the device, and the sampled ids come back to the host."""
    import torch
    from kvcache_b200 import LLM, EngineOptions, SamplingParams
    options = EngineOptions(dtype="bfloat16", page_size=16, max_cached_tokens=batch * (context + 64), max_running=batch,
                            max_tokens_per_step=2048, chunk_size=2048, max_model_len=context + 64, use_graphs=True)
    llm = LLM(folder, options)
    # The prompts are prefilled one after the other under the token budget, so the requests start to decode a
    # few steps apart; none may finish inside the timed region (the batch would shrink), and the longest ends
    # at `context` tokens.
    lead = 4 * batch
    prompt_len = context - steps - warmup - lead
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, llm.core.model.vocab_size, (prompt_len,), generator=g).tolist() for _ in range(batch)]
    for p in prompts:
        llm.scheduler.add_request(p, SamplingParams(max_new_tokens=steps + warmup + 2 * lead, ignore_eos=True))
    while any(r.num_computed < len(r.prompt) for r in llm.scheduler.running) or llm.scheduler.waiting:
        llm.step()                                   # prefill, untimed
    for _ in range(warmup):
        llm.step()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with clocks.region("e2e"):
        wall = time.perf_counter()
        begin.record()
        for _ in range(steps):
            llm.step()                               # plans and launches a step, reads the tokens of the one before
        end.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - wall
    if len(llm.scheduler.running) != batch or llm.scheduler.stats.finished:
        raise RuntimeError("a request finished inside the timed region: the steps did not all decode the whole batch")
    ms = max(begin.elapsed_time(end), wall * 1e3)
    h2d = llm.core.runner.last_h2d_bytes
    d2h = batch * 4
    del llm
    torch.cuda.empty_cache()
    return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "h2d": h2d, "d2h": d2h}


def time_published_workload(folder, clocks):
    """The workload of the reference's published number - one request, a prompt of 29 tokens, 256 new tokens -
    timed as the reference times it (apps/qwen_infer.cu:30-38,194-209): wall clock of every decode step with
    the copies of the token to the device and back, the first 16 steps left out, the median."""
    import torch
    from kvcache_b200 import LLM, EngineOptions, SamplingParams
    llm = LLM(folder, EngineOptions(dtype="bfloat16", page_size=16, max_cached_tokens=1024, max_running=1,
                                    max_tokens_per_step=64, chunk_size=64, max_model_len=1024, use_graphs=True))
    prompt = torch.randint(0, llm.core.model.vocab_size, (PUBLISHED_PROMPT,), generator=torch.Generator().manual_seed(6)).tolist()
    llm.pipelined = False                            # a step's token is read before the next step is planned, as there
    llm.scheduler.add_request(prompt, SamplingParams(max_new_tokens=PUBLISHED_NEW, ignore_eos=True))
    llm.step()                                       # the prompt
    times = []
    with clocks.region("published_workload"):
        while llm.has_work():
            t = time.perf_counter()
            llm.step()
            times.append((time.perf_counter() - t) * 1e6)
    times = sorted(times[16:])
    del llm
    torch.cuda.empty_cache()
    return {"median_us": times[len(times) // 2], "steps": len(times)}


def run_ours(args) -> int:
    import torch  # noqa: F401
    peaks = load_peaks()
    clocks = ClockSampler().start()
    with tempfile.TemporaryDirectory() as tmp:
        folder = make_folder(tmp, args.layers)
        main_run = time_decode(folder, args.batch, args.context, args.steps, args.warmup, clocks, "decode", use_graphs=not args.no_graphs)
        points = {}
        if not args.skip_points:
            for b in (1, 64):
                points[f"decode_b{b}"] = round(time_decode(folder, b, CONTEXT, args.steps, args.warmup, clocks, f"decode_b{b}")["tok_s"], 1)
            published = time_published_workload(folder, clocks)
            points["b1_prompt29_new256_us_per_tok"] = round(published["median_us"], 1)
            points["b1_prompt29_new256"] = round(1e6 / published["median_us"], 1)
        prefill = {"ms": float("nan"), "tok_s": float("nan"), "flops": float("nan")} if args.skip_prefill else \
            time_prefill(folder, PREFILL_TOKENS, clocks)
        e2e = None if args.skip_e2e else time_e2e(folder, args.batch, args.context, args.steps, args.warmup, clocks)
        kernels = None if args.skip_kernels else time_kernel_classes(folder, args.batch, args.context, peaks)
    clocks.stop()

    achieved = main_run["bytes_per_step"] / (main_run["ms_per_step"] / 1e3) / 1e9
    headline_clocks = dict(clocks.regions.get("decode", {}), how=clocks.how,
                           regions={k: v for k, v in clocks.regions.items() if k != "decode"})
    line = {
        "metric": METRIC if (args.batch, args.context) == (8, CONTEXT) else f"decode tok/s at batch {args.batch} (Qwen2.5-0.5B shape, context {args.context})",
        "value": round(main_run["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["ms_per_step"], 4), "ms_per_step_p50": round(main_run["ms_p50"], 4),
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(points["b1_prompt29_new256"] / PUBLISHED_TOK_S, 2) if "b1_prompt29_new256" in points else None,
        "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": dict(bench_config(args.batch, args.layers, args.steps, args.warmup, peaks["source"]), seq_len=args.context),
        "prefill": {"value": round(prefill["tok_s"], 1), "tokens": PREFILL_TOKENS, "ms": round(prefill["ms"], 3),
                    "frac": round(prefill["flops"] / (prefill["ms"] / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points, "clocks": headline_clocks, "gpu_launches": main_run["launches"],
    }
    if kernels:
        line["roofline"]["kernels"] = kernels
    if e2e is not None:
        line["e2e"] = {"value": round(e2e["tok_s"], 1), "unit": "tok/s", "ms_per_step": round(e2e["ms_per_step"], 4),
                       "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"]}
    print(json.dumps(line))
    return 0


def run_reference(args) -> int:
    """The same workload through the unmodified reference.  Its `qwen_serve` prints no timing, so the decode
    time is the difference between two runs of the same eight requests that differ only in the number of new
    tokens (`warmup` and `warmup + steps` decode steps each), taken between its own two lines on standard error
    (after the weights are loaded, after the last step).  Host token ids in, host token ids out: the number is
    the end-to-end number too."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import torch
        import reference_arm as ra
        if args.gpus != 1:
            raise ra.ReferenceUnavailable("the reference runs on one GPU")
        if not torch.cuda.is_available():
            raise ra.ReferenceUnavailable("no CUDA device")
        ra.programs()
        steps, warmup = min(args.steps, REFERENCE_MAX_STEPS), max(args.warmup, 3)
        batch = args.batch
        clocks = ClockSampler(interval=0.02).start()
        with tempfile.TemporaryDirectory() as tmp:
            folder = make_folder(tmp, QWEN25_05B["num_hidden_layers"])
            weights = ra.export_weights(folder, os.path.join(tmp, "reference_weights"))
            g = torch.Generator().manual_seed(4)
            vocab = QWEN25_05B["vocab_size"]
            prompt_len = CONTEXT - steps - warmup - 1
            prompts = [torch.randint(0, vocab, (prompt_len,), generator=g).tolist() for _ in range(batch)]
            # qwen_serve runs max_new - 1 decode steps for a request (its first token comes from the prompt).
            with clocks.region("decode"):
                ids_short, t_short, steps_short = ra.run_serve(weights, [(warmup + 1, p) for p in prompts])
                ids_long, t_long, steps_long = ra.run_serve(weights, [(warmup + steps + 1, p) for p in prompts])
            decoded = sum(len(i) for i in ids_long) - sum(len(i) for i in ids_short)
            if decoded != batch * steps or t_long <= t_short:
                raise ra.ReferenceUnavailable(f"qwen_serve decoded {decoded} tokens more in the longer run, {batch * steps} expected "
                                              "(an end token among the random model's choices?)")
            if any(a != b[:len(a)] for a, b in zip(ids_short, ids_long)):
                raise ra.ReferenceUnavailable("qwen_serve generated different tokens in two runs of the same requests")
            seconds = t_long - t_short
            live = min(batch, ra.SERVE_MAX_BATCH, ra.SERVE_POOL_PAGES // -(-CONTEXT // ra.SERVE_PAGE))
            points = {}
            with clocks.region("decode_b1"):
                new = steps + 17
                _, b1 = ra.run_infer(weights, torch.randint(0, vocab, (CONTEXT - new,), generator=g).tolist(), new, graph=True)
            points["decode_b1"] = round(1e6 / b1["median_us"], 1)
            with clocks.region("published_workload"):
                _, pub = ra.run_infer(weights, torch.randint(0, vocab, (PUBLISHED_PROMPT,), generator=g).tolist(), PUBLISHED_NEW, graph=True)
            points["b1_prompt29_new256_us_per_tok"] = round(pub["median_us"], 1)
            points["b1_prompt29_new256"] = round(1e6 / pub["median_us"], 1)
        clocks.stop()
        value = batch * steps / seconds
        # Per decode step of n requests the reference copies ids, positions and lengths (4 n bytes each), n + 1 offsets
        # and the block tables of the n requests to the device and n ids back (apps/qwen_serve.cu:143-147,173).
        pages = -(-CONTEXT // ra.SERVE_PAGE)
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
            "ms_per_step": round(seconds / steps * 1e3, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": round(points["b1_prompt29_new256"] / PUBLISHED_TOK_S, 2), "dtype": "fp16", "data": "synthetic",
            "impl": "reference", "config": bench_config(batch, QWEN25_05B["num_hidden_layers"], steps, warmup, load_peaks()["source"]),
            "points": points,
            "how": {"program": "qwen_serve, unmodified, nvcc sm_100a", "requests_live_at_a_time": live,
                    "decode_steps_of_the_program": [steps_short, steps_long], "seconds": [round(t_short, 3), round(t_long, 3)],
                    "timing": "difference of two runs between the program's own lines on standard error"},
            "clocks": dict(clocks.regions.get("decode", {}), how=clocks.how,
                           regions={k: v for k, v in clocks.regions.items() if k != "decode"}),
            "e2e": {"value": round(value, 2), "unit": "tok/s", "ms_per_step": round(seconds / steps * 1e3, 3),
                    "h2d_bytes_per_step": live * 12 + (live + 1) * 4 + live * pages * 4, "d2h_bytes_per_step": live * 4},
        }
        print(json.dumps(line))
        return 0
    except Exception as exc:                         # the arm must end with its line and exit 0
        reason = str(exc).splitlines()[0] if str(exc) else type(exc).__name__
        print(json.dumps({"impl": "reference", "unavailable": reason[:300]}))
        return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--layers", type=int, default=QWEN25_05B["num_hidden_layers"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=CONTEXT, help="tokens each request has cached while it decodes")
    parser.add_argument("--skip-e2e", action="store_true")
    parser.add_argument("--skip-points", action="store_true")
    parser.add_argument("--skip-prefill", action="store_true")
    parser.add_argument("--skip-kernels", action="store_true")
    parser.add_argument("--no-graphs", action="store_true", help="launch the decode step's kernels one by one (for profilers)")
    args = parser.parse_args()

    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py measures a one-GPU engine: --gpus {args.gpus} is not supported (this build has no multi-GPU path)")
        return 2
    args.warmup = max(args.warmup, 3)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
