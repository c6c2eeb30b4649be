"""Load-time request caps chosen from estimated parameter bytes vs device memory.

``aggressive`` allows 32 concurrent requests and 1024 new tokens per request, ``stable`` one request
and 256 tokens (reference: vllm/engine/loadtime_policy.py:15-132).  On a 180 GB B200 almost every
supported checkpoint lands in ``aggressive``; the stable tier remains for models that fill the GPU.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class LoadtimePolicy:
    name: str
    max_concurrent_requests: int
    max_tokens_cap: int
    reason: str = ""


AGGRESSIVE = LoadtimePolicy("aggressive", 32, 1024, "model fits with ample KV head-room")
STABLE = LoadtimePolicy("stable", 1, 256, "model leaves little memory for KV cache")
UNCAPPED = LoadtimePolicy("uncapped", 1 << 30, 1 << 30, "explicitly disabled")


def estimate_param_bytes(model) -> int:
    total = 0
    seen = set()
    for t in list(model.parameters()) + list(model.buffers()):
        if t.data_ptr() in seen:
            continue
        seen.add(t.data_ptr())
        total += t.numel() * t.element_size()
    return total


def select_loadtime_policy(param_bytes: int, device_total_bytes: int | None, mode: str = "auto",
                           stable_fraction: float = 0.80) -> LoadtimePolicy:
    mode = (mode or "auto").lower()
    if mode in ("aggressive", "stable"):
        return AGGRESSIVE if mode == "aggressive" else STABLE
    if mode in ("off", "none", "uncapped"):
        return UNCAPPED
    if not device_total_bytes or device_total_bytes <= 0:
        return AGGRESSIVE
    if param_bytes >= stable_fraction * device_total_bytes:
        return STABLE
    return AGGRESSIVE
