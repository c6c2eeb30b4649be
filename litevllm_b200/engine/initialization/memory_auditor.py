"""Start-up memory report: parameter and buffer bytes by dtype, packed int4 / GGUF payload bytes,
KV pool bytes and (on a GPU) what the allocator holds.
Reference: vllm/engine/initialization/memory_auditor.py."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class MemorySnapshot:
    param_bytes_by_dtype: dict[str, int] = field(default_factory=dict)
    buffer_bytes_by_dtype: dict[str, int] = field(default_factory=dict)
    quantized_bytes: int = 0        # packed int4 codes + scales/zeros, raw GGUF blocks
    kv_cache_bytes: int = 0
    device_allocated_bytes: int | None = None
    device_reserved_bytes: int | None = None

    @property
    def weight_bytes(self) -> int:
        return sum(self.param_bytes_by_dtype.values()) + sum(self.buffer_bytes_by_dtype.values()) + self.quantized_bytes

    def as_dict(self) -> dict:
        return {"params": dict(self.param_bytes_by_dtype), "buffers": dict(self.buffer_bytes_by_dtype),
                "quantized_bytes": self.quantized_bytes, "kv_cache_bytes": self.kv_cache_bytes,
                "weight_bytes": self.weight_bytes, "device_allocated_bytes": self.device_allocated_bytes,
                "device_reserved_bytes": self.device_reserved_bytes}

    def report(self) -> str:
        gib = 2 ** 30
        parts = [f"{k}: {v / gib:.2f} GiB" for k, v in sorted(self.param_bytes_by_dtype.items()) if v]
        if self.quantized_bytes:
            parts.append(f"quantized payload: {self.quantized_bytes / gib:.2f} GiB")
        parts.append(f"KV pool: {self.kv_cache_bytes / gib:.2f} GiB")
        if self.device_allocated_bytes is not None:
            parts.append(f"device allocated: {self.device_allocated_bytes / gib:.2f} GiB")
        return ", ".join(parts)


class MemoryAuditor:
    QUANT_ATTRS = ("int4", "gguf_weight", "raw_weight")

    @staticmethod
    def _tensor_bytes(obj, seen: set[int]) -> int:
        total = 0
        if isinstance(obj, torch.Tensor):
            if obj.data_ptr() not in seen:
                seen.add(obj.data_ptr())
                total += obj.numel() * obj.element_size()
        elif isinstance(obj, (list, tuple)):
            for o in obj:
                total += MemoryAuditor._tensor_bytes(o, seen)
        elif isinstance(obj, dict):
            for o in obj.values():
                total += MemoryAuditor._tensor_bytes(o, seen)
        elif obj is not None and hasattr(obj, "__dict__") and not isinstance(obj, torch.nn.Module):
            for o in vars(obj).values():
                total += MemoryAuditor._tensor_bytes(o, seen)
        return total

    def snapshot(self, model: torch.nn.Module, kv_cache=None, device: torch.device | None = None) -> MemorySnapshot:
        snap = MemorySnapshot()
        seen: set[int] = set()
        for p in model.parameters():
            if p.data_ptr() in seen:
                continue
            seen.add(p.data_ptr())
            k = str(p.dtype).replace("torch.", "")
            snap.param_bytes_by_dtype[k] = snap.param_bytes_by_dtype.get(k, 0) + p.numel() * p.element_size()
        for b in model.buffers():
            if b.data_ptr() in seen:
                continue
            seen.add(b.data_ptr())
            k = str(b.dtype).replace("torch.", "")
            snap.buffer_bytes_by_dtype[k] = snap.buffer_bytes_by_dtype.get(k, 0) + b.numel() * b.element_size()
        for m in model.modules():
            for name in self.QUANT_ATTRS:
                snap.quantized_bytes += self._tensor_bytes(getattr(m, name, None), seen)
        if kv_cache is not None:
            snap.kv_cache_bytes = int(getattr(kv_cache, "total_bytes", 0))
        if device is not None and device.type == "cuda":
            snap.device_allocated_bytes = int(torch.cuda.memory_allocated(device))
            snap.device_reserved_bytes = int(torch.cuda.memory_reserved(device))
        return snap
