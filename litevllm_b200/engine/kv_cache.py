"""Flat paged KV pool: ONE contiguous device buffer carved into per-layer K and V views
``[num_blocks, n_kv_heads, block_size, head_dim]`` (per-layer shapes may differ, e.g. Gemma4's
sliding vs global layers).  fp8 caches are e4m3 with per-tensor scales kept in the inference
config.  Reference: vllm/engine/initialization/flat_kv_cache_allocator.py:47-140 (layout there is
[blocks, block, kv_heads, head_dim]; the head-major order here gives each (block, head) a
contiguous ``block_size x head_dim`` tile for bulk loads).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..utils.misc import dtype_nbytes


@dataclass(frozen=True)
class KVLayerSpec:
    num_kv_heads: int
    head_dim: int
    v_head_dim: int | None = None     # MLA-style caches may use another width for V (0 = no V)

    @property
    def v_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim


def kv_torch_dtype(kv_cache_dtype: str, model_dtype: torch.dtype) -> torch.dtype:
    name = (kv_cache_dtype or "auto").lower()
    if name in ("auto", "fp16", "bf16", "model"):
        return model_dtype if model_dtype in (torch.float16, torch.bfloat16, torch.float32) else torch.bfloat16
    if name in ("fp8", "fp8_e4m3"):
        return torch.float8_e4m3fn
    if name == "turbo_int4":
        # packed-int4 KV is a unified-memory capacity feature of the reference; on a 180 GB part the
        # fp8 cache is the compact format, so the request maps to it.
        return torch.float8_e4m3fn
    raise ValueError(f"unknown kv cache dtype {kv_cache_dtype!r}")


def bytes_per_block(specs: list[KVLayerSpec], block_size: int, dtype: torch.dtype) -> int:
    e = dtype_nbytes(dtype)
    return sum(s.num_kv_heads * block_size * (s.head_dim + s.v_dim) * e for s in specs)


class FlatKVCache:
    def __init__(self, specs: list[KVLayerSpec], num_blocks: int, block_size: int,
                 dtype: torch.dtype, device: torch.device):
        self.specs, self.num_blocks, self.block_size = specs, num_blocks, block_size
        self.dtype, self.device = dtype, device
        e = dtype_nbytes(dtype)
        offsets, total = [], 0
        for s in specs:
            kb = num_blocks * s.num_kv_heads * block_size * s.head_dim * e
            vb = num_blocks * s.num_kv_heads * block_size * s.v_dim * e
            kb_al = (kb + 255) // 256 * 256
            vb_al = (vb + 255) // 256 * 256
            offsets.append((total, kb, total + kb_al, vb))
            total += kb_al + vb_al
        self.total_bytes = total
        self.buffer = torch.zeros(max(total, 1), dtype=torch.uint8, device=device)
        self.layers: list[tuple[torch.Tensor, torch.Tensor]] = []
        for s, (ko, kb, vo, vb) in zip(specs, offsets):
            k = self.buffer[ko:ko + kb].view(dtype).view(num_blocks, s.num_kv_heads, block_size, s.head_dim)
            v = self.buffer[vo:vo + vb].view(dtype).view(num_blocks, s.num_kv_heads, block_size, s.v_dim) \
                if s.v_dim > 0 else k[:, :, :, :0]
            self.layers.append((k, v))

    def __getitem__(self, i: int):
        return self.layers[i]

    def __len__(self) -> int:
        return len(self.layers)

    def copy_blocks_out(self, block_ids: list[int]) -> list[tuple[torch.Tensor, torch.Tensor]]:
        idx = torch.tensor(block_ids, dtype=torch.long, device=self.device)
        return [(k.index_select(0, idx), v.index_select(0, idx)) for k, v in self.layers]

    def copy_blocks_in(self, block_ids: list[int], saved) -> None:
        idx = torch.tensor(block_ids, dtype=torch.long, device=self.device)
        for (k, v), (sk, sv) in zip(self.layers, saved):
            k.index_copy_(0, idx, sk[: len(block_ids)])
            if v.numel():
                v.index_copy_(0, idx, sv[: len(block_ids)])
