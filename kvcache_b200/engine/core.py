"""Model, cache manager, kernel set and step function of one engine, made from a model folder
and the engine's options.  Generation, the command lines and trace replay all stand on this."""
from __future__ import annotations

from typing import Optional

import torch

from ..cache.manager import CacheManager
from ..cache.pages import pages_for
from ..config.options import EngineOptions
from .loading import load_model
from .runner import ModelRunner


class EngineCore:
    def __init__(self, folder: str, options: EngineOptions, kernels=None):
        self.options = options
        self.device = torch.device(options.device)
        if kernels is None:
            from ..kernels.api import CudaKernels   # raises if the device or the compiler is missing
            kernels = CudaKernels(self.device)
        self.kernels = kernels
        config_len = None
        self.model = None
        from ..config.registry import load_config
        self.config = load_config(folder)
        config_len = int(getattr(self.config, "max_position_embeddings", 0)) or None
        max_len = options.max_model_len or config_len
        if config_len is not None and max_len > config_len:
            raise ValueError(f"max_model_len {max_len} exceeds the model's max_position_embeddings {config_len}")
        if options.num_pages is not None:
            num_pages = options.num_pages
        elif options.max_cached_tokens is not None:
            num_pages = pages_for(options.max_cached_tokens, options.page_size)
        else:
            raise ValueError("give the cache a size: EngineOptions.num_pages or max_cached_tokens")
        max_len = min(max_len, num_pages * options.page_size)
        self.max_model_len = max_len
        self.model = load_model(folder, options.dtype, self.device, max_positions=max_len, strict=options.strict_weights)
        self.cache = CacheManager(self.model.cache_entries(), page_size=options.page_size, num_pages=num_pages,
                                  max_slots=options.max_running, max_tokens_per_request=max_len,
                                  dtype=options.dtype, device=self.device)
        self.runner = ModelRunner(self.model, self.cache, self.kernels,
                                  max_tokens_per_step=options.max_tokens_per_step,
                                  max_segments=options.max_running, use_graphs=options.use_graphs)
