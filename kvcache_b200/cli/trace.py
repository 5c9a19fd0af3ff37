"""Trace replay: feeds given token ids through the model step by step and writes logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--page-size P] [--max-live L]

Standard input carries one JSON object a line,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
All entries of a step run as one batch through the engine's own step function, cache and
kernels (nothing here computes).  For a step in which logits are wanted the file
`<out>/<step>.f32` receives them as little-endian float32 [wanted, vocab], in the order of
the entries and of `want`; after every step the line `done <step>` is printed and flushed.
The reference has no such program; its nearest relatives compare generated ids
(tools/run_serve.py:45-49, tools/diff_cudagraph.py:20-68).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict

PAGE_SIZE = 16          # default of --page-size; divides 64, the rounding of --max-tokens
MAX_LIVE_REQUESTS = 8   # default of --max-live


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens that live requests hold at any time (each rounded up to 64)")
    parser.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens in a page of the cache (a power of two)")
    parser.add_argument("--max-live", type=int, default=MAX_LIVE_REQUESTS, help="most requests that are live at a time")
    args = parser.parse_args(argv)

    import numpy as np
    import torch
    from ..config.options import EngineOptions
    from ..engine.core import EngineCore
    from ..engine.runner import StepEntry

    os.makedirs(args.out, exist_ok=True)
    unit = max(64, args.page_size)                       # a request's tokens are rounded up to this
    capacity = max(unit, (args.max_tokens + unit - 1) // unit * unit)
    options = EngineOptions(dtype=args.dtype, page_size=args.page_size, max_cached_tokens=capacity,
                            max_running=args.max_live, max_tokens_per_step=capacity, use_graphs=False)
    core = EngineCore(args.model, options)
    slots: Dict[str, int] = {}

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for item in record.get("entries", []):
            key = str(item["id"])
            if key not in slots:
                slots[key] = core.cache.admit()
            entries.append(StepEntry(slots[key], item["tokens"], item.get("want", [])))
        if entries:
            logits = core.runner.step(entries)
            if logits.shape[0] > 0:
                host = logits.detach().to("cpu", torch.float32).contiguous().numpy()
                host.astype("<f4", copy=False).tofile(os.path.join(args.out, f"{step}.f32"))
            else:
                torch.cuda.synchronize(core.device)
            core.kernels.check_errors()
        for key in record.get("end", []):
            slot = slots.pop(str(key), None)
            if slot is not None:
                core.cache.release(slot)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
