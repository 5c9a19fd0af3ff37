"""Slots for per-request state of fixed size.

Every live request holds one slot: the row of its block tables and the index of its
state in each layer's state tensor.  The architecture built here keeps no state between
steps besides keys and values, so its state tensors are empty; a mixer that declares a
`StateSpec` gets `[slots, *shape]`, zeroed when a request is admitted.
"""
from __future__ import annotations

from typing import List

import numpy as np


class OutOfSlots(RuntimeError):
    pass


class SlotAllocator:
    def __init__(self, num_slots: int):
        if num_slots < 1:
            raise ValueError("at least one slot is needed")
        self.num_slots = num_slots
        self._free: List[int] = list(range(num_slots - 1, -1, -1))
        self._held = np.zeros(num_slots, dtype=bool)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfSlots(f"all {self.num_slots} request slots are in use")
        slot = self._free.pop()
        self._held[slot] = True
        return slot

    def free(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots or not self._held[slot]:
            raise ValueError(f"slot {slot} is not in use")
        self._held[slot] = False
        self._free.append(slot)

    def is_held(self, slot: int) -> bool:
        return 0 <= slot < self.num_slots and bool(self._held[slot])
