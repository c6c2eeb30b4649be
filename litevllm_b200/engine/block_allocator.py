"""Paged-KV block id allocator.  Ids 1..N-1 are allocatable; id 0 is the permanent null block that
pads block tables and is never written (reference: vllm/engine/block_allocator.py:8-49).

A step allocates or frees a handful of ids, so a deque plus a set is all this needs; the block
tables themselves live on the device (``kv_block_manager``).
"""
from __future__ import annotations

from collections import deque


class BlockAllocator:
    def __init__(self, num_blocks: int):
        if num_blocks < 2:
            raise ValueError("need at least the null block and one usable block")
        self.num_blocks = num_blocks
        self._free: deque[int] = deque(range(1, num_blocks))
        self._used: set[int] = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return len(self._used)

    def can_allocate(self, n: int) -> bool:
        return n <= len(self._free)

    def allocate(self, n: int = 1) -> list[int]:
        if n > len(self._free):
            raise MemoryError(f"KV cache exhausted: want {n} blocks, {len(self._free)} free")
        out = [self._free.popleft() for _ in range(n)]
        self._used.update(out)
        return out

    def free(self, block_ids) -> None:
        for b in block_ids:
            if b == 0:
                continue
            if b not in self._used:
                raise ValueError(f"double free or foreign block id {b}")
            self._used.remove(b)
            self._free.append(b)

    def reset(self) -> None:
        self._free = deque(range(1, self.num_blocks))
        self._used.clear()
