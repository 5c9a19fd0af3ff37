"""Shared helpers of the tests: building an engine over a kernel set, random prompts."""
from __future__ import annotations

import random
from typing import List

import torch


def make_runner(folder: str, kernels, *, dtype: str, device: str, page_size: int, num_pages: int,
                max_slots: int = 4, max_tokens_per_step: int = 512, max_tokens_per_request: int = 512):
    from kvcache_b200.cache import CacheManager
    from kvcache_b200.engine.loading import load_model
    from kvcache_b200.engine.runner import ModelRunner
    model = load_model(folder, dtype=dtype, device=device, max_positions=max_tokens_per_request)
    cache = CacheManager(model.cache_entries(), page_size=page_size, num_pages=num_pages, max_slots=max_slots,
                         max_tokens_per_request=max_tokens_per_request, dtype=dtype, device=device)
    return ModelRunner(model, cache, kernels, max_tokens_per_step=max_tokens_per_step)


def random_tokens(vocab: int, n: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]
