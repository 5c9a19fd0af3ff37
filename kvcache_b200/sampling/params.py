"""Per-request sampling parameters.  The reference decodes greedily for `max_new` tokens
and stops at two fixed end ids (apps/qwen_serve.cu:23, :182-190); temperature and seed are
this engine's additions."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class SamplingParams:
    max_new_tokens: int = 32
    temperature: float = 0.0            # 0: greedy (lowest index wins a tie)
    seed: int = 0                       # keys the request's random stream
    eos_token_ids: Optional[Tuple[int, ...]] = None   # None: the configuration's
    ignore_eos: bool = False

    def __post_init__(self) -> None:
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
