"""A pool of page ids: free list, reference counts (src/kv/block_pool.cpp:7-43).

A fresh pool hands out the lowest id first; a released page is the next one handed out.
Misuse (releasing a free page, retaining a free page, an id outside the pool) raises.
"""
from __future__ import annotations

from ..errors import CapacityError, InvalidArgument


class BlockPool:
    def __init__(self, num_blocks: int):
        if num_blocks <= 0:
            raise InvalidArgument(f"a block pool needs at least one block, got {num_blocks}")
        self._refs = [0] * num_blocks
        self._free = list(range(num_blocks - 1, -1, -1))  # stack: lowest id on top

    @property
    def num_blocks(self) -> int:
        return len(self._refs)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def _check(self, block: int) -> None:
        if not 0 <= block < len(self._refs):
            raise InvalidArgument(f"block id {block} outside [0, {len(self._refs)})")

    def ref_count(self, block: int) -> int:
        self._check(block)
        return self._refs[block]

    def allocate(self) -> int:
        if not self._free:
            raise CapacityError(f"KV cache is full: all {len(self._refs)} blocks are in use")
        block = self._free.pop()
        self._refs[block] = 1
        return block

    def retain(self, block: int) -> None:
        self._check(block)
        if self._refs[block] == 0:
            raise InvalidArgument(f"cannot retain free block {block}")
        self._refs[block] += 1

    def release(self, block: int) -> None:
        self._check(block)
        if self._refs[block] == 0:
            raise InvalidArgument(f"block {block} released while already free")
        self._refs[block] -= 1
        if self._refs[block] == 0:
            self._free.append(block)
