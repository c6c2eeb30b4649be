"""Named runtime profiles: ``auto`` (= ``balanced``), ``balanced``, ``latency``, ``throughput``,
``accuracy``, ``benchmark``.  A profile fixes KV dtype, block size, slot count and scheduling
knobs; model adapters may override parts of it afterwards.
Defaults and per-profile overrides follow vllm/engine/runtime_profile.py:35-180 of the reference,
except that the default KV dtype on B200 is the model dtype ("auto") rather than packed int4.
"""
from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass, field, replace
from types import MappingProxyType
from typing import Any

from .runtime_policy import BackendRuntimePolicy, SchedulerRuntimePolicy

SUPPORTED_PROFILE_NAMES = ("auto", "balanced", "latency", "throughput", "accuracy", "benchmark")
SERVICE_PROFILE_NAMES = ("balanced", "latency", "throughput")
DEFAULT_ACTIVE_REQUESTS = 4


def freeze(value: Any) -> Any:
    if isinstance(value, Mapping):
        return MappingProxyType({k: freeze(v) for k, v in value.items()})
    if isinstance(value, (list, tuple)):
        return tuple(freeze(v) for v in value)
    if isinstance(value, (set, frozenset)):
        return frozenset(freeze(v) for v in value)
    return value


@dataclass(frozen=True)
class RuntimeProfile:
    requested_name: str
    effective_name: str
    description: str
    kv_cache_dtype: str = "auto"
    block_size: int = 16
    kv_max_model_len: int | None = None
    kv_max_active_requests: int = DEFAULT_ACTIVE_REQUESTS
    fusion_level: int = 2
    enable_decode_priority: bool = True
    prefill_chunk_size: int = 0            # 0 = choose from the model policy
    prefill_reserved_tokens: int = 0
    prefill_reserve_backlog: int = 2
    prefill_catchup_ratio: float = 0.25
    prefill_microbatch_size: int = 8
    min_prefill_chunk_size: int = 128
    max_prefill_chunk_size: int | None = None
    prefill_sla_ttft_ms: float = 2000.0
    default_min_new_tokens: int = 0
    queue_timeout_s: float = 30.0
    async_driver_min_step_interval_s: float = 0.0002
    memory_audit_topn: int = 20
    k_scale: float = 1.0
    v_scale: float = 1.0
    use_prompt_guard: bool = True
    scheduler_policy: SchedulerRuntimePolicy = field(default_factory=SchedulerRuntimePolicy)
    backend_policy: BackendRuntimePolicy = field(default_factory=BackendRuntimePolicy)
    model_policy: Mapping[str, Any] = field(default_factory=dict)
    kernel_policy: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        object.__setattr__(self, "model_policy", freeze(self.model_policy))
        object.__setattr__(self, "kernel_policy", freeze(self.kernel_policy))

    def stats(self) -> dict[str, Any]:
        return {
            "requested": self.requested_name, "effective": self.effective_name,
            "description": self.description, "kv_cache_dtype": self.kv_cache_dtype,
            "block_size": self.block_size, "kv_max_model_len": self.kv_max_model_len,
            "kv_max_active_requests": self.kv_max_active_requests, "fusion_level": self.fusion_level,
            "async_driver_min_step_interval_s": self.async_driver_min_step_interval_s,
        }


_GREEDY_ON = BackendRuntimePolicy(gpu_greedy_sampling=True)

_OVERRIDES: dict[str, dict[str, Any]] = {
    "balanced": dict(description="general serving: decode priority with prefill catch-up",
                     backend_policy=_GREEDY_ON),
    "latency": dict(description="single active request, short context, lowest time per token",
                    kv_max_active_requests=1, kv_max_model_len=512, backend_policy=_GREEDY_ON),
    "throughput": dict(description="many active requests, larger prefill micro-batches",
                       kv_max_active_requests=16, prefill_microbatch_size=32),
    "accuracy": dict(description="fp8 KV cache, no lossy shortcuts", kv_cache_dtype="fp8"),
    "benchmark": dict(description="benchmark harness defaults", backend_policy=_GREEDY_ON),
}


class RuntimeProfileRegistry:
    @classmethod
    def names(cls) -> tuple[str, ...]:
        return SUPPORTED_PROFILE_NAMES

    @classmethod
    def resolve_from_config(cls, config) -> RuntimeProfile:
        return cls.resolve(requested_profile=config.profile, kv_type=getattr(config, "kv_type", "auto"))

    @classmethod
    def resolve(cls, requested_profile: str | None = "auto", kv_type: str = "auto") -> RuntimeProfile:
        requested = str(requested_profile or "auto").strip().lower()
        if requested not in SUPPORTED_PROFILE_NAMES:
            raise ValueError(f"Unsupported runtime profile {requested!r}; expected one of "
                             f"{', '.join(SUPPORTED_PROFILE_NAMES)}")
        effective = "balanced" if requested == "auto" else requested
        profile = RuntimeProfile(requested_name=requested, effective_name=effective,
                                 **_OVERRIDES[effective])
        if kv_type and kv_type != "auto":
            profile = replace(profile, kv_cache_dtype=kv_type)
        return profile
