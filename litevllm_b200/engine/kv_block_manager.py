"""Per-request block lists on top of :class:`BlockAllocator`, plus the persistent device block
table ``int32 [max_active, blocks_per_seq]`` that attention kernels index by request slot.

``ensure_blocks`` is grow-only and is called before a step for the number of tokens the step will
have in cache afterwards.  Rows are padded with the null block 0.  Dirty rows are uploaded in one
pinned-memory copy per step.  Reference: vllm/engine/kv_block_manager.py:13-195.
"""
from __future__ import annotations

import torch

from ..utils.misc import cdiv
from .block_allocator import BlockAllocator


class KVBlockManager:
    def __init__(self, allocator: BlockAllocator, block_size: int, max_active: int,
                 blocks_per_seq: int, device: torch.device, kv_cache=None):
        self.allocator = allocator
        self.block_size = block_size
        self.max_active = max_active
        self.blocks_per_seq = blocks_per_seq
        self.device = device
        self.kv_cache = kv_cache
        self._blocks: dict[str, list[int]] = {}
        self._slot_of: dict[str, int] = {}
        pin = device.type == "cuda"
        self.host_table = torch.zeros(max_active, blocks_per_seq, dtype=torch.int32, pin_memory=pin)
        self.block_tables = torch.zeros(max_active, blocks_per_seq, dtype=torch.int32, device=device)
        self._dirty: set[int] = set()

    # ------------------------------------------------------------------ queries
    def blocks_of(self, request_id: str) -> list[int]:
        return self._blocks.get(request_id, [])

    def num_blocks_needed(self, request_id: str, num_tokens: int) -> int:
        return max(0, cdiv(num_tokens, self.block_size) - len(self._blocks.get(request_id, [])))

    def can_grow(self, request_id: str, num_tokens: int) -> bool:
        return self.allocator.can_allocate(self.num_blocks_needed(request_id, num_tokens))

    # ------------------------------------------------------------------ lifecycle
    def register(self, request_id: str, slot_idx: int) -> None:
        self._blocks.setdefault(request_id, [])
        self._slot_of[request_id] = slot_idx
        self.host_table[slot_idx].zero_()
        self._dirty.add(slot_idx)

    def ensure_blocks(self, request_id: str, num_tokens: int) -> list[int]:
        """Make sure the request owns blocks for ``num_tokens`` tokens; returns newly added ids."""
        have = self._blocks.setdefault(request_id, [])
        need = cdiv(num_tokens, self.block_size)
        if need > self.blocks_per_seq:
            raise ValueError(f"request {request_id} needs {need} blocks > per-sequence cap {self.blocks_per_seq}")
        if need <= len(have):
            return []
        new = self.allocator.allocate(need - len(have))
        slot = self._slot_of.get(request_id)
        if slot is not None:
            start = len(have)
            self.host_table[slot, start:start + len(new)] = torch.tensor(new, dtype=torch.int32)
            self._dirty.add(slot)
        have.extend(new)
        return new

    def release(self, request_id: str) -> None:
        blocks = self._blocks.pop(request_id, None)
        slot = self._slot_of.pop(request_id, None)
        if blocks:
            self.allocator.free(blocks)
        if slot is not None:
            self.host_table[slot].zero_()
            self._dirty.add(slot)

    def flush(self) -> None:
        """Upload dirty block-table rows (call once before launching a step)."""
        if not self._dirty:
            return
        rows = sorted(self._dirty)
        self._dirty.clear()
        if len(rows) > self.max_active // 2 or self.device.type != "cuda":
            self.block_tables.copy_(self.host_table, non_blocking=True)
            return
        lo, hi = rows[0], rows[-1] + 1
        self.block_tables[lo:hi].copy_(self.host_table[lo:hi], non_blocking=True)

    # ------------------------------------------------------------------ prefix cache support
    def capture_prefix(self, request_id: str, num_tokens: int):
        """Clone the blocks covering the first ``num_tokens`` tokens (whole blocks only)."""
        n = num_tokens // self.block_size
        ids = self._blocks.get(request_id, [])[:n]
        if not ids or self.kv_cache is None:
            return None
        return self.kv_cache.copy_blocks_out(ids)

    def materialize_prefix(self, request_id: str, saved, num_blocks: int) -> int:
        """Allocate ``num_blocks`` blocks for the request and fill them from a captured prefix."""
        self.ensure_blocks(request_id, num_blocks * self.block_size)
        ids = self._blocks[request_id][:num_blocks]
        self.kv_cache.copy_blocks_in(ids, saved)
        return num_blocks * self.block_size

    def stats(self) -> dict:
        return {"free_blocks": self.allocator.num_free, "used_blocks": self.allocator.num_used,
                "block_size": self.block_size, "tracked_requests": len(self._blocks)}
