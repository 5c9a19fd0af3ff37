"""Time per class of kernel, behind a flag: CUDA events around every operator of the kernel set.

The reference times whole decode steps by wall clock (apps/qwen_infer.cu:30-38) and has no
per-kernel figures.  `KernelTiming` wraps the operators of a `CudaKernels` object while it is
switched on: each call is bracketed by two events on the launching stream and filed under a
class - the operator's name, and for matrix products the weight's shape, since one operator
serves the q/k/v, output, feed-forward and head products.  With each class go the bytes its
calls had to move (weights, activations, the keys and values of the step's requests), so that a
report can state microseconds, GB/s and launches per class.

A kernel between two events neither starts before its predecessor has ended nor overlaps its
successor, which the engine's launch chain otherwise allows; the classes therefore add up to
more than a step takes.  CUDA graphs cannot hold these events: switch graphs off while timing.

Launched one by one, the kernels of a decode step take the host longer to launch (about 12 us
each) than the GPU to run, and an event pair around an idle GPU measures the host.  So the
first operator of every step (`embed`) is preceded by a kernel that only spins for `hold_ms`
milliseconds: while it runs the host queues the step's launches, and the events then see the
kernels back to back.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Tuple

import torch


def _numel_bytes(t) -> int:
    return 0 if t is None else t.numel() * t.element_size()


def _attention_bytes(batch, kv, num_heads: int) -> int:
    """Keys and values of the step's requests (every key once per kv head), queries in, results out."""
    spec = kv.spec
    element = kv.k_pages.element_size()
    host = batch.host
    if "starts" in host and "counts" in host:
        keys = int((host["starts"] + host["counts"]).sum())
        if spec.window:
            keys = int(sum(min(int(s + c), spec.window + int(c) - 1) for s, c in zip(host["starts"], host["counts"])))
    else:
        keys = batch.max_kv_len * batch.num_segments
    rows = batch.num_tokens * num_heads * spec.head_dim * element
    return 2 * keys * spec.num_kv_heads * spec.head_dim * element + 2 * rows


class KernelTiming:
    OPERATORS = ("embed", "add_rmsnorm", "silu_mul", "gate_up_act", "linear", "qkv_rope_append", "rope_append_attention",
                 "paged_attention", "sample")

    def __init__(self, kernels, hold_ms: float = 4.0):
        self.kernels = kernels
        self.hold_cycles = int(hold_ms * 1e-3 * getattr(torch.cuda.get_device_properties(kernels.device), "clock_rate", 1_900_000) * 1e3) if hold_ms > 0 else 0
        self.records: List[tuple] = []      # (class, bytes, begin event, end event, launches)
        self._saved: Dict[str, Callable] = {}
        self._depth = 0

    # ---- which class a call belongs to and what it has to move -----------------------------------
    @staticmethod
    def _describe(name: str, args, kwargs) -> Tuple[str, int]:
        if name == "linear":
            x, w, out = args[0], args[1], args[2]
            return f"linear {w.shape[0]}x{w.shape[1]}", _numel_bytes(w) + _numel_bytes(x) + _numel_bytes(out)
        if name == "gate_up_act":
            x, w, out = args[0], args[1], args[2]
            return f"gate_up_act {w.shape[0]}x{w.shape[1]}", _numel_bytes(w) + _numel_bytes(x) + _numel_bytes(out)
        if name == "embed":
            out = args[2]
            return name, out.numel() * (4 + args[0].element_size())
        if name == "add_rmsnorm":
            h, delta, out = args[0], args[1], args[4]
            rows, width = out.shape
            return name, rows * width * (8 + out.element_size() + (delta.element_size() if delta is not None else 0))
        if name == "silu_mul":
            return name, _numel_bytes(args[0]) + _numel_bytes(args[1])
        if name == "qkv_rope_append":
            return name, 2 * _numel_bytes(args[0])
        if name == "rope_append_attention":
            qkv, batch, kv, num_heads = args[0], args[4], args[5], args[7]
            return name, _attention_bytes(batch, kv, num_heads) + _numel_bytes(qkv)
        if name == "paged_attention":
            batch, kv, num_heads = args[1], args[2], args[4]
            return name, _attention_bytes(batch, kv, num_heads)
        if name == "sample":
            return name, _numel_bytes(args[0])
        return name, 0

    # ---- switching on and off -------------------------------------------------------------------------
    def start(self) -> None:
        for name in self.OPERATORS:
            original = getattr(self.kernels, name, None)
            if original is None:
                continue
            self._saved[name] = original
            setattr(self.kernels, name, self._wrap(name, original))

    def _wrap(self, name: str, original: Callable) -> Callable:
        def timed(*args, **kwargs):
            if self._depth:                              # called by an operator that is being timed: part of its class
                return original(*args, **kwargs)
            label, nbytes = self._describe(name, args, kwargs)
            if name == "embed" and self.hold_cycles:
                torch.cuda._sleep(self.hold_cycles)      # keeps the GPU busy while the host queues this step
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            launches = self.kernels.launches
            begin.record()
            self._depth += 1
            try:
                result = original(*args, **kwargs)
            finally:
                self._depth -= 1
            end.record()
            if name == "rope_append_attention" and result is False:
                return result                            # nothing ran: the caller makes the two calls
            self.records.append((label, nbytes, begin, end, self.kernels.launches - launches))
            return result
        return timed

    def stop(self) -> Dict[str, dict]:
        """Restores the operators; returns {class: {"us", "bytes", "calls", "launches"}} summed over all calls."""
        for name in self._saved:
            try:
                delattr(self.kernels, name)              # the wrapper lives on the instance; the class method is back
            except AttributeError:
                pass
        self._saved.clear()
        torch.cuda.synchronize(self.kernels.device)
        report: Dict[str, dict] = {}
        for label, nbytes, begin, end, launches in self.records:
            entry = report.setdefault(label, {"us": 0.0, "bytes": 0, "calls": 0, "launches": 0})
            entry["us"] += begin.elapsed_time(end) * 1e3
            entry["bytes"] += nbytes
            entry["calls"] += 1
            entry["launches"] += launches
        self.records.clear()
        return report


def format_report(report: Dict[str, dict], steps: int = 1) -> str:
    """A table of the classes, slowest first: microseconds a step, share, GB/s."""
    total = sum(e["us"] for e in report.values()) or 1.0
    lines = [f"{'class':<34}{'us/step':>10}{'share':>8}{'calls':>7}{'GB/s':>9}"]
    for label, e in sorted(report.items(), key=lambda kv: -kv[1]["us"]):
        gbs = e["bytes"] / (e["us"] * 1e-6) / 1e9 if e["us"] > 0 and e["bytes"] else 0.0
        lines.append(f"{label:<34}{e['us'] / steps:>10.1f}{100 * e['us'] / total:>7.1f}%{e['calls'] // max(steps, 1):>7}{gbs:>9.0f}")
    return "\n".join(lines)
