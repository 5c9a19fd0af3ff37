"""Chooses next tokens on the device from float32 logits: greedy, or Gumbel-max sampling at a
temperature with a counter-based random stream per request (see csrc/sampling.cu).  The
reference's sampler is a greedy argmax kernel (src/qwen_kernels.cu:229-248)."""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from .params import SamplingParams


class Sampler:
    def __init__(self, kernels, device: torch.device | str, vocab_size: int, max_rows: int):
        self.kernels = kernels
        self.device = torch.device(device)
        self.vocab_size = vocab_size
        self.max_rows = max_rows
        parts = kernels.sample_parts(vocab_size)
        pin = self.device.type == "cuda"
        # One packed host buffer per call: [temperature f32 | counter i32 | seed i64] by rows.
        self._host = torch.zeros(max_rows * 4, dtype=torch.int32, pin_memory=pin)
        self._dev = torch.zeros(max_rows * 4, dtype=torch.int32, device=self.device)
        self._scratch_val = torch.empty(max_rows * parts, dtype=torch.float32, device=self.device)
        self._scratch_idx = torch.empty(max_rows * parts, dtype=torch.int32, device=self.device)
        self._out = torch.empty(max_rows, dtype=torch.int32, device=self.device)
        self._out_host = torch.empty(max_rows, dtype=torch.int32, pin_memory=pin)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], counters: Sequence[int]) -> np.ndarray:
        """One token per row of `logits`; `counters[r]` is how many tokens row r's request has
        sampled before (it counts the request's random stream).  Returns host int32 [R]."""
        R = logits.shape[0]
        if R == 0:
            return np.zeros(0, dtype=np.int32)
        if R > self.max_rows:
            raise ValueError(f"{R} rows to sample; the sampler was made for {self.max_rows}")
        host = self._host.numpy()
        host[:R].view(np.float32)[:] = [p.temperature for p in params]
        host[R:2 * R] = counters
        host[2 * R:4 * R].view(np.int64)[:] = [p.seed & 0x7FFFFFFFFFFFFFFF for p in params]
        self._dev[:4 * R].copy_(self._host[:4 * R], non_blocking=True)
        dev = self._dev
        self.kernels.sample(logits, dev[:R].view(torch.float32), dev[2 * R:4 * R].view(torch.int64), dev[R:2 * R],
                            self._out[:R], self._scratch_val, self._scratch_idx)
        self._out_host[:R].copy_(self._out[:R], non_blocking=True)
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()
        return self._out_host[:R].numpy().copy()
