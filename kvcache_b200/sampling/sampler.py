"""Brings sampled tokens to the host.  The choice itself - greedy, or Gumbel-max sampling at a
temperature with a counter-based random stream per request - is made on the device by the
step function (csrc/sampling.cu); the reference's sampler is a greedy argmax kernel whose
result is copied back every step (src/qwen_kernels.cu:229-248, apps/qwen_serve.cu:172-174)."""
from __future__ import annotations

import numpy as np
import torch


class TokenReader:
    def __init__(self, device: torch.device | str, max_rows: int):
        self.device = torch.device(device)
        self._host = torch.empty(max_rows, dtype=torch.int32, pin_memory=self.device.type == "cuda")

    def read(self, tokens: torch.Tensor) -> np.ndarray:
        """Device int32 [R] -> host numpy int32 [R]; waits for the step that produced them."""
        R = tokens.shape[0]
        self._host[:R].copy_(tokens, non_blocking=True)
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()
        return self._host[:R].numpy().copy()
