"""Benchmark of kvcache_b200: decode tokens a second of the Qwen2.5-0.5B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on standard output.  `value`: decoded tokens a second at batch 8 and the
benchmark context (device-timed decode steps through the engine's step function and device
sampler); `e2e`: the same through the Python entry point (`LLM.step`: host token ids in,
host token ids out, scheduler and copies included); `prefill`: one 2,048-token prompt;
`roofline`: bytes a decode step has to read (every weight once, the cache of the live
requests) over its time, against the measured copy bandwidth; `points`: decode at batch 1
and 64.  Weights are seeded random numbers of the named shape, prompts are random ids, and
the cache of the timed requests is filled with random keys and values instead of being
prefilled (`data`: synthetic).
"""
from __future__ import annotations

import argparse
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
PUBLISHED_TOK_S = 1e6 / 8104.0     # the reference's best published decode: 8,104 us/token (RTX 3060, batch 1)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


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
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            fields = [f.strip() for f in line.split(",")]
            if len(fields) < 6:
                continue
            try:
                clocks.append(int(fields[0]))
                max_clock = int(fields[1])
            except ValueError:
                continue
            for name, value in zip(names, fields[2:6]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


def make_folder(tmp: str, layers: int) -> str:
    import torch
    import kvcache_b200  # noqa: F401
    from kvcache_b200.config import config_from_dict
    from kvcache_b200.weights import write_random_model
    config = dict(QWEN25_05B, num_hidden_layers=layers, max_window_layers=layers)
    return write_random_model(os.path.join(tmp, "qwen25_05b_random"), config_from_dict(config), seed=0, dtype=torch.bfloat16)


def fill_cache_randomly(core, slots, context):
    """Gives each slot `context` cached tokens of random keys and values (no prefill run)."""
    import torch
    core.cache.extend([(s, context) for s in slots])
    g = torch.Generator(device=core.device).manual_seed(1)
    for group in core.cache.groups:
        group.k_pool.normal_(0.0, 1.0, generator=g)
        group.v_pool.normal_(0.0, 1.0, generator=g)


def time_decode(folder, batch, context, steps, warmup, use_graphs=True, sampler=None):
    """Device-timed decode steps at `batch` requests of about `context` cached tokens each."""
    import torch
    from kvcache_b200.config.options import EngineOptions
    from kvcache_b200.engine.core import EngineCore
    from kvcache_b200.engine.decode_loop import DecodeLoop
    options = EngineOptions(dtype="bfloat16", page_size=16, max_cached_tokens=batch * (context + 16), max_running=batch,
                            max_tokens_per_step=max(batch, 16), max_model_len=context + 16, use_graphs=use_graphs)
    core = EngineCore(folder, options)
    slots = [core.cache.admit() for _ in range(batch)]
    start_len = context - steps - warmup
    fill_cache_randomly(core, slots, start_len)
    loop = DecodeLoop(core, slots, use_graphs=use_graphs)
    tokens = torch.randint(0, core.model.vocab_size, (batch,), generator=torch.Generator().manual_seed(2), dtype=torch.int32)
    loop.set_tokens(tokens)
    for _ in range(warmup):
        loop.step()
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.start()                               # clocks are sampled during the timed region only
        time.sleep(0.05)
    launches_before = loop.launches
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        loop.step()
    end.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler is not None else None
    core.kernels.check_errors()
    ms = begin.elapsed_time(end)
    mean_context = start_len + warmup + (steps - 1) / 2.0 + 1
    step_bytes = core.model.decode_weight_bytes() + batch * mean_context * core.cache.kv_bytes_per_token()
    result = {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "bytes_per_step": step_bytes,
              "launches": loop.launches - launches_before, "clocks": clocks}
    del loop, core
    torch.cuda.empty_cache()
    return result


def time_prefill(folder, tokens, layers_total, repeats=3, warm=5):
    import torch
    from kvcache_b200.config.options import EngineOptions
    from kvcache_b200.engine.core import EngineCore
    from kvcache_b200.engine.runner import StepEntry
    options = EngineOptions(dtype="bfloat16", page_size=16, max_cached_tokens=tokens + 16, max_running=1,
                            max_tokens_per_step=tokens, max_model_len=tokens + 16, use_graphs=True)
    core = EngineCore(folder, options)
    ids = torch.randint(0, core.model.vocab_size, (tokens,), generator=torch.Generator().manual_seed(3)).tolist()
    times = []
    for i in range(warm + repeats):                  # the step is replayed from a graph once its shape has come a few times
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


def time_e2e(folder, batch, context, steps, warmup):
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
    wall = time.perf_counter()
    begin.record()
    for _ in range(steps):
        llm.step()                                   # plans and launches a step, reads the tokens of the one before
    end.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall
    if len(llm.scheduler.running) != batch or llm.scheduler.stats.finished:
        raise RuntimeError("a request finished inside the timed region: the steps did not all decode the whole batch")
    ms = max(begin.elapsed_time(end), wall * 1e3)
    h2d = llm.core.runner.last_h2d_bytes
    d2h = batch * 4
    return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "h2d": h2d, "d2h": d2h}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--layers", type=int, default=QWEN25_05B["num_hidden_layers"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--skip-e2e", action="store_true")
    parser.add_argument("--skip-points", action="store_true")
    parser.add_argument("--skip-prefill", action="store_true")
    parser.add_argument("--no-graphs", action="store_true", help="launch the decode step's kernels one by one (for profilers)")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "pip cannot install kimxinw/kvcache: the tree has neither "
                          "setup.py nor pyproject.toml (a CMake project of CUDA executables with sizes compiled in)"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures a one-GPU engine: --gpus {args.gpus} is not supported (this build has no multi-GPU path)")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch
    peaks = load_peaks()
    with tempfile.TemporaryDirectory() as tmp:
        folder = make_folder(tmp, args.layers)
        main_run = time_decode(folder, args.batch, CONTEXT, args.steps, args.warmup, use_graphs=not args.no_graphs,
                               sampler=ClockSampler())
        clocks = main_run["clocks"]
        points = {}
        if not args.skip_points:
            for b in (1, 64):
                points[f"decode_b{b}"] = round(time_decode(folder, b, CONTEXT, args.steps, args.warmup)["tok_s"], 1)
        prefill = {"ms": float("nan"), "tok_s": float("nan"), "flops": float("nan")} if args.skip_prefill else \
            time_prefill(folder, PREFILL_TOKENS, args.layers)
        e2e = None if args.skip_e2e else time_e2e(folder, args.batch, CONTEXT, args.steps, args.warmup)

    achieved = main_run["bytes_per_step"] / (main_run["ms_per_step"] / 1e3) / 1e9
    c = QWEN25_05B
    line = {
        "metric": "decode tok/s at batch 8 (Qwen2.5-0.5B shape, bf16, context 4096)",
        "value": round(main_run["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(main_run["tok_s"] / PUBLISHED_TOK_S, 2), "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": "Qwen2.5-0.5B shape, random weights", "global_batch": args.batch, "seq_len": CONTEXT,
                   "parallelism": "single GPU", "layers": args.layers, "layers_of_model": c["num_hidden_layers"],
                   "hidden": c["hidden_size"], "q_heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"],
                   "head_dim": c["hidden_size"] // c["num_attention_heads"], "intermediate": c["intermediate_size"],
                   "vocab": c["vocab_size"], "page_size": 16, "new_tokens": args.steps + args.warmup,
                   "prefill_tokens": PREFILL_TOKENS, "l2": "inputs larger than L2 (weights read once per step)",
                   "peaks": peaks["source"]},
        "prefill": {"value": round(prefill["tok_s"], 1), "tokens": PREFILL_TOKENS, "ms": round(prefill["ms"], 3),
                    "frac": round(prefill["flops"] / (prefill["ms"] / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points, "clocks": clocks, "gpu_launches": main_run["launches"],
    }
    if e2e is not None:
        line["e2e"] = {"value": round(e2e["tok_s"], 1), "unit": "tok/s", "ms_per_step": round(e2e["ms_per_step"], 4),
                       "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"]}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
