"""Options of the engine itself (not of the model): what the reference fixes as
BLOCK, NUM_BLOCKS and MAXB (apps/qwen_serve.cu:21) and `EngineConfig`
(src/include/engine.h:24-30) become fields here."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

DTYPE_NAMES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32"}


def canonical_dtype(name: str) -> str:
    try:
        return DTYPE_NAMES[name.lower()]
    except KeyError:
        raise ValueError(f"dtype must be one of bfloat16, float32; got '{name}'") from None


@dataclass
class EngineOptions:
    dtype: str = "bfloat16"
    page_size: int = 16                    # tokens in a page of the cache
    num_pages: Optional[int] = None        # pages of each cache group; None: from max_cached_tokens
    max_cached_tokens: Optional[int] = None  # pool capacity in tokens when num_pages is None
    max_running: int = 8                   # live requests (state slots, rows of the block table)
    max_tokens_per_step: int = 2048        # token budget of one step
    chunk_size: int = 2048                 # largest portion of one prompt in a step (measured: 512 tokens cost 1.5 ms, 2048 cost 2.9 ms)
    max_model_len: Optional[int] = None    # None: the configuration's max_position_embeddings
    admission: str = "reserve"             # "reserve" (worst case held back) or "optimistic" (preempts)
    use_graphs: bool = True                # CUDA graphs for steps of decoded tokens and of one portion of one prompt
    seed: int = 0
    device: str = "cuda:0"
    strict_weights: bool = True            # False: tensors of the folder that the model does not use are no error

    def __post_init__(self) -> None:
        self.dtype = canonical_dtype(self.dtype)
        if self.page_size < 1 or (self.page_size & (self.page_size - 1)) != 0:
            raise ValueError(f"page_size must be a power of two, got {self.page_size}")
        if self.admission not in ("reserve", "optimistic"):
            raise ValueError(f"admission must be 'reserve' or 'optimistic', got '{self.admission}'")
        if self.max_running < 1 or self.max_tokens_per_step < 1 or self.chunk_size < 1:
            raise ValueError("max_running, max_tokens_per_step and chunk_size must be positive")
