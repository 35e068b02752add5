"""Slots of per-request state of fixed size, beside the paged cache.

A mixer that carries state across steps (a recurrence, a running sum) declares a shape; every
admitted request owns one slot index, the same in every such layer. A slot is taken when a
request is admitted (its first `CacheManager.reserve`), zeroed as it is handed out, and given
back when the request ends or is preempted: state is recomputed from token 0 like the keys
and values. A request that waits holds none. The reference has no such state (src/engine/sequence.h:15-30); with
no stateful mixer in the model the pool holds indices only and no memory.
"""
from __future__ import annotations

from ..errors import CapacityError, InvalidArgument


class StateSlots:
    def __init__(self, needs, max_requests: int, device=None):
        """needs[i]: parts.StateNeed or None per run entry."""
        if max_requests <= 0:
            raise InvalidArgument(f"state slots need a positive request count, got {max_requests}")
        self.max_requests = max_requests
        self._free = list(range(max_requests - 1, -1, -1))
        self._used = [False] * max_requests
        self._tensors = {}
        self.has_state = any(need is not None for need in needs)
        if device is not None:
            import torch
            for i, need in enumerate(needs):
                if need is not None:
                    self._tensors[i] = torch.zeros((max_requests, *need.shape), dtype=need.dtype, device=device)
        self.bytes_per_slot = sum(t[0].numel() * t.element_size() for t in self._tensors.values())

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise CapacityError(f"all {self.max_requests} state slots are in use")
        slot = self._free.pop()
        self._used[slot] = True
        self.zero(slot)
        return slot

    def release(self, slot: int) -> None:
        if not 0 <= slot < self.max_requests or not self._used[slot]:
            raise InvalidArgument(f"state slot {slot} released while free")
        self._used[slot] = False
        self._free.append(slot)

    def zero(self, slot: int) -> None:
        for t in self._tensors.values():
            t[slot].zero_()

    def tensor(self, entry: int):
        return self._tensors.get(entry)
