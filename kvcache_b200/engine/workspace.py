"""Named scratch buffers that outlive a step: activations keep their addresses from step
to step (which CUDA graphs need) and nothing is allocated once the sizes have been seen.
The reference allocates its activation buffers once, sized for the longest prompt
(apps/qwen_serve.cu:69-83)."""
from __future__ import annotations

from typing import Dict, Tuple

import torch


class Workspace:
    def __init__(self, device: torch.device | str, row_capacity: int = 0):
        """`row_capacity`: buffers whose first dimension is at most this many rows are made
        for that many rows at once, so they never move afterwards."""
        self.device = torch.device(device)
        self.row_capacity = row_capacity
        self._buffers: Dict[str, torch.Tensor] = {}
        self._views: Dict[tuple, torch.Tensor] = {}      # (name, shape, dtype) -> the view handed out last time
        self.moved = 0        # how many times an existing buffer was replaced by a larger one
        self.frozen = False   # set while a CUDA graph is captured or replayed: growing is an error

    def buffer(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        key = (name, tuple(shape), dtype)
        view = self._views.get(key)
        if view is not None:
            return view                                  # the same request as before: nothing to compute or to slice
        count = 1
        for s in shape:
            count *= int(s)
        buf = self._buffers.get(name)
        if buf is None or buf.dtype != dtype or buf.numel() < count:
            if self.frozen:
                raise RuntimeError(f"workspace buffer '{name}' would have to grow to {count} elements "
                                   f"while its addresses are pinned by a CUDA graph")
            capacity = max(count, 1)
            if shape and 0 < int(shape[0]) <= self.row_capacity:
                capacity = max(capacity, count // int(shape[0]) * self.row_capacity)
            if buf is not None and buf.dtype == dtype:
                capacity = max(capacity, buf.numel())
            if buf is not None:
                self.moved += 1
            buf = torch.empty(capacity, dtype=dtype, device=self.device)
            self._buffers[name] = buf
            for old in [k for k in self._views if k[0] == name]:
                del self._views[old]                     # views of the buffer that was replaced
        view = buf[:count].view(shape)
        self._views[key] = view
        return view

    def zeros(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """Like `buffer`, but zero when first made (or remade); its users leave it zero."""
        count = 1
        for s in shape:
            count *= int(s)
        before = self._buffers.get(name)
        view = self.buffer(name, shape, dtype)
        if self._buffers[name] is not before:
            self._buffers[name].zero_()
        return view

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())
