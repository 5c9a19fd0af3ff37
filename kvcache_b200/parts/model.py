"""A decoder model as data: parts, and the order in which its layers run.

The reference's model is the body of two lambdas (apps/qwen_serve.cu:90-124 and
:127-175).  Here the same sequence - embedding, layers, final norm on the wanted
rows, output matrix with float32 logits - runs over a list of `LayerCall`s, which
may name a layer twice or let a call read the cache another call wrote.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ..weights.loader import TensorSpec
from .base import (TORCH_DTYPES, Block, LayerContext, Norm, PagedKVSpec, PositionEncoding, StateSpec,
                   StepBatch)


@dataclass(frozen=True)
class LayerCall:
    layer: int                 # index into the model's blocks
    cache: int                 # which cache entry the call uses
    writes_cache: bool = True  # False: reads what the writer of that entry stored in this step


@dataclass(frozen=True)
class CacheEntry:
    """What one cache id needs: pages of keys and values and/or per-request state."""
    kv: Optional[PagedKVSpec]
    state: Any                     # None, a StateSpec, or {name: StateSpec}


class DecoderModel:
    def __init__(self, *, config: Any, dtype: str, vocab_size: int, width: int, embed_name: str,
                 head_name: Optional[str], blocks: Sequence[Block], schedule: Sequence[LayerCall],
                 final_norm: Norm, position: Optional[PositionEncoding] = None, ignorable_tensors: Sequence[str] = ()):
        self.config = config
        self.dtype_name = dtype
        self.dtype = TORCH_DTYPES[dtype]
        self.vocab_size, self.width = vocab_size, width
        self.embed_name, self.head_name = embed_name, head_name
        self.blocks = list(blocks)
        self.schedule = list(schedule)
        self.final_norm = final_norm
        self.position = position
        # Names (shell patterns) of tensors that checkpoints of this architecture may carry without the model using them.
        self.ignorable_tensors = tuple(ignorable_tensors)
        self._fold_cache: Dict[tuple, bool] = {}
        self.embed: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self.device: Optional[torch.device] = None
        for call in self.schedule:
            if not 0 <= call.layer < len(self.blocks):
                raise ValueError(f"schedule names layer {call.layer}; the model has {len(self.blocks)} blocks")
        writers = {}
        for call in self.schedule:
            if call.writes_cache:
                if call.cache in writers:
                    raise ValueError(f"cache entry {call.cache} is written by two calls of the schedule")
                writers[call.cache] = call.layer
            elif call.cache not in writers:
                raise ValueError(f"a call reads cache entry {call.cache} before any call writes it")
        ids = sorted(writers)
        if ids != list(range(len(ids))):
            raise ValueError(f"cache entries must be numbered 0..n-1, got {ids}")
        self._writers = writers

    # ---- weights -----------------------------------------------------------
    @property
    def tied(self) -> bool:
        return self.head_name is None

    def _parts(self):
        out = list(self.blocks) + [self.final_norm]
        if self.position is not None:
            out.append(self.position)
        return out

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs: Dict[str, TensorSpec] = {self.embed_name: TensorSpec((self.vocab_size, self.width))}
        if self.head_name is not None:
            specs[self.head_name] = TensorSpec((self.vocab_size, self.width))
        for part in self._parts():
            specs.update(part.tensor_specs())
        return specs

    def init_kinds(self) -> Dict[str, str]:
        kinds: Dict[str, str] = {}
        for part in self._parts():
            kinds.update(part.init_kinds())
        return kinds

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device | str) -> None:
        device = torch.device(device)
        self.device = device
        self.embed = tensors[self.embed_name].to(self.dtype).to(device).contiguous()
        # A tied output matrix is the embedding table itself: one buffer, read twice
        # (the reference stores the alias twice, tools/dump_weights.py:24-26).
        self.head = self.embed if self.head_name is None else \
            tensors[self.head_name].to(self.dtype).to(device).contiguous()
        for part in self._parts():
            part.bind(tensors, device)

    def decode_weight_bytes(self) -> int:
        """Bytes of weights a decode step reads once: every layer call's block, the final
        norm and the output matrix (embedding rows are a gather, not a stream)."""
        total = sum(self.blocks[c.layer].weight_bytes() for c in self.schedule)
        return total + self.final_norm.weight_bytes() + self.head.numel() * self.head.element_size()

    # ---- cache needs -------------------------------------------------------
    def cache_entries(self) -> List[CacheEntry]:
        entries = []
        for cache_id in range(len(self._writers)):
            mixer = self.blocks[self._writers[cache_id]].mixer
            entries.append(CacheEntry(mixer.cache_spec(), mixer.state_spec()))
        return entries

    def step_planners(self, kernels: Any) -> List[Any]:
        """The planners of all mixers' kernels, each once (by name), in the order of the blocks."""
        found: Dict[str, Any] = {}
        for block in self.blocks:
            for planner in block.mixer.step_planners(kernels):
                found.setdefault(planner.name, planner)
        return list(found.values())

    def _folds(self, kernels: Any, num_rows: int) -> bool:
        """Whether a step of `num_rows` rows runs every layer in its folded form: all layers must offer it, and nothing
        may change the embedded rows behind the back of their rounded copy."""
        if self.position is not None and type(self.position).on_embed is not PositionEncoding.on_embed:
            return False
        key = (id(kernels), num_rows, getattr(kernels, "fold_key", None))
        found = self._fold_cache.get(key)
        if found is None:
            found = self._fold_cache[key] = all(self.blocks[call.layer].supports_fold(kernels, num_rows) for call in self.schedule)
        return found

    # ---- one step ----------------------------------------------------------
    def forward(self, batch: StepBatch, kernels: Any, workspace: Any, cache: Any) -> torch.Tensor:
        """Runs the rows of `batch` through the layer calls; returns float32 logits
        [batch.num_wanted, vocab] for `batch.wanted_rows`."""
        T, R = batch.num_tokens, batch.num_wanted
        h = workspace.buffer("model.h", (T, self.width), torch.float32)
        # Steps of few rows take every layer's folded form, if every layer offers one: the residual stream then also
        # exists rounded to the compute type (`h16`), norms run inside the products after them and adds inside the
        # products before them.
        fold = self._folds(kernels, T)
        h16 = workspace.buffer("model.h16", (T, self.width), self.dtype) if fold else None
        if fold:
            kernels.embed(self.embed, batch.token_ids, h, batch.token_src, batch.last_tokens, h16)
        else:
            kernels.embed(self.embed, batch.token_ids, h, batch.token_src, batch.last_tokens)
        base = LayerContext(batch=batch, kernels=kernels, workspace=workspace)
        if self.position is not None:
            self.position.on_embed(h, base)
        pending = None
        for index, call in enumerate(self.schedule):
            ctx = LayerContext(batch=batch, kernels=kernels, workspace=workspace,
                               kv=cache.kv_view(call.cache, call.writes_cache),
                               state=cache.state(call.cache), call_index=index)
            if fold:
                self.blocks[call.layer].forward_folded(h, h16, ctx)
            else:
                pending = self.blocks[call.layer].forward(h, pending, ctx)
        logits = workspace.buffer("model.logits", (R, self.vocab_size), torch.float32)
        if R > 0:
            normed = workspace.buffer("model.final", (R, self.width), self.dtype)
            self.final_norm.add_norm(h, pending, normed, base, rows=batch.wanted_rows)
            kernels.linear(normed, self.head, logits)
        return logits
