"""Flat paged KV pool: ONE contiguous device buffer carved into per-layer K and V views
``[num_blocks, n_kv_heads, block_size, head_dim]`` (per-layer shapes may differ, e.g. Gemma4's
sliding vs global layers).  Formats: 16-bit; e4m3 with per-tensor scales kept in the inference
config (``fp8``); e4m3 with one fp32 scale per (token, head) row (``fp8_block``: block-scaled fp8);
packed int4 rows ``[.., head_dim / 2]`` bytes with one fp32 scale per row (``turbo_int4``).  The
row-scaled formats carry their scale pools ``[num_blocks, n_kv_heads, block_size]`` as attributes of
the K / V views (``.fi_scales``, ``.fi_mode``), which is what the op layer looks for.  Reference: vllm/engine/initialization/flat_kv_cache_allocator.py:47-140 (layout there is
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
    if name in ("fp8_block", "fp8_row"):
        return torch.float8_e4m3fn
    if name == "turbo_int4":
        return torch.uint8
    raise ValueError(f"unknown kv cache dtype {kv_cache_dtype!r}")


def kv_format(kv_cache_dtype: str) -> int:
    """0 = 16-bit, 1 = fp8 with per-tensor scales, 2 = fp8 with a scale per (token, head) row, 3 = packed int4
    with a scale per row."""
    name = (kv_cache_dtype or "auto").lower()
    return {"fp8": 1, "fp8_e4m3": 1, "fp8_block": 2, "fp8_row": 2, "turbo_int4": 3}.get(name, 0)


def bytes_per_block(specs: list[KVLayerSpec], block_size: int, dtype: torch.dtype, fmt: int = 0) -> int:
    e = dtype_nbytes(dtype)
    div = 2 if fmt == 3 else 1
    row_scales = 8 if fmt >= 2 else 0           # one fp32 scale per K row and per V row
    return sum(s.num_kv_heads * block_size * ((s.head_dim + s.v_dim) * e // div + row_scales) for s in specs)


class FlatKVCache:
    def __init__(self, specs: list[KVLayerSpec], num_blocks: int, block_size: int,
                 dtype: torch.dtype, device: torch.device, fmt: int = 0):
        self.specs, self.num_blocks, self.block_size = specs, num_blocks, block_size
        self.dtype, self.device, self.fmt = dtype, device, fmt
        e = dtype_nbytes(dtype)
        div = 2 if fmt == 3 else 1             # packed int4: two channels per byte
        offsets, total = [], 0
        for s in specs:
            if fmt == 3 and (s.head_dim % 32 or s.v_dim % 32):
                raise ValueError("packed-int4 KV needs head dimensions that are multiples of 32")
            kb = num_blocks * s.num_kv_heads * block_size * s.head_dim * e // div
            vb = num_blocks * s.num_kv_heads * block_size * s.v_dim * e // div
            kb_al = (kb + 255) // 256 * 256
            vb_al = (vb + 255) // 256 * 256
            offsets.append((total, kb, total + kb_al, vb))
            total += kb_al + vb_al
        self.total_bytes = total
        self.buffer = torch.zeros(max(total, 1), dtype=torch.uint8, device=device)
        self.layers: list[tuple[torch.Tensor, torch.Tensor]] = []
        self.scale_bytes = 0
        for s, (ko, kb, vo, vb) in zip(specs, offsets):
            k = self.buffer[ko:ko + kb].view(dtype).view(num_blocks, s.num_kv_heads, block_size, s.head_dim // div)
            v = self.buffer[vo:vo + vb].view(dtype).view(num_blocks, s.num_kv_heads, block_size, s.v_dim // div) \
                if s.v_dim > 0 else k[:, :, :, :0]
            if fmt >= 2:
                for t in (k, v):
                    t.fi_scales = torch.zeros(num_blocks, s.num_kv_heads, block_size, dtype=torch.float32, device=device)
                    t.fi_mode = fmt
                    self.scale_bytes += t.fi_scales.numel() * 4
            self.layers.append((k, v))
        self.total_bytes += self.scale_bytes

    def __getitem__(self, i: int):
        return self.layers[i]

    def __len__(self) -> int:
        return len(self.layers)

    def copy_blocks_out(self, block_ids: list[int]) -> list[tuple[torch.Tensor, torch.Tensor]]:
        """Clones of the given blocks of every layer (row scales ride along as ``.fi_scales`` of the clones)."""
        idx = torch.tensor(block_ids, dtype=torch.long, device=self.device)
        out = []
        for k, v in self.layers:
            ck, cv = k.index_select(0, idx), v.index_select(0, idx)
            if self.fmt >= 2:
                ck.fi_scales, cv.fi_scales = k.fi_scales.index_select(0, idx), v.fi_scales.index_select(0, idx)
            out.append((ck, cv))
        return out

    def copy_blocks_in(self, block_ids: list[int], saved) -> None:
        idx = torch.tensor(block_ids, dtype=torch.long, device=self.device)
        n = len(block_ids)
        for (k, v), (sk, sv) in zip(self.layers, saved):
            k.index_copy_(0, idx, sk[:n])
            if v.numel():
                v.index_copy_(0, idx, sv[:n])
            if self.fmt >= 2:
                k.fi_scales.index_copy_(0, idx, sk.fi_scales[:n])
                v.fi_scales.index_copy_(0, idx, sv.fi_scales[:n])
