"""A decode loop that stays on the device: the tokens one step samples are the next step's
input without a trip to the host.  The host only advances lengths and block tables, which
do not depend on the sampled values, so it can queue step n+1 while step n runs.  This is
what the benchmark times as the decode step proper; generation with end conditions goes
through `LLM.step`, which reads every step's tokens."""
from __future__ import annotations

from typing import Sequence

import torch

from .core import EngineCore
from .runner import StepEntry


class DecodeLoop:
    def __init__(self, core: EngineCore, slots: Sequence[int], temperature: float = 0.0, seed: int = 0,
                 use_graphs: bool = True):
        self.core = core
        self.slots = list(slots)
        self.temperature, self.seed = temperature, seed
        self.runner = core.runner
        self.runner.use_graphs = use_graphs and core.device.type == "cuda"
        self._count = 0

    @property
    def launches(self) -> int:
        return self.core.kernels.launches

    def set_tokens(self, tokens: torch.Tensor) -> None:
        """The first step's input ids, placed where a previous step would have left its samples."""
        self.runner.last_tokens[:len(self.slots)].copy_(tokens.to(self.core.device, torch.int32))

    def step(self) -> torch.Tensor:
        """One token for every slot; returns the device tensor of the tokens just sampled."""
        entries = [StepEntry(slot, (0,), (0,), (self.temperature, self.seed + i, self._count), token_from_last=i)
                   for i, slot in enumerate(self.slots)]
        _, tokens = self.runner.step(entries, sample=True)
        self._count += 1
        return tokens
