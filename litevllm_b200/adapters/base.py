"""Model adapters: per-family capabilities and runtime policy, chosen before the model loads.
Reference: vllm/adapters/base.py:26-70."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class ModelCapabilities:
    supports_lora: bool = True
    supports_multimodal: bool = False
    supports_chunked_prefill: bool = True
    supports_prefix_cache: bool = True
    supports_sampling: bool = True       # False: greedy only (token-returning executors)
    supports_cuda_graph: bool = True


@dataclass(frozen=True)
class RuntimeModelPolicy:
    force_kv_cache_dtype: str | None = None
    prefill_chunk_size: int = 0
    admission_cap: int | None = None
    tuning_overrides: dict[str, str] = field(default_factory=dict)
    model_policy: dict[str, Any] = field(default_factory=dict)
    kernel_policy: dict[str, Any] = field(default_factory=dict)
    verified_decode_batch_sizes: tuple[int, ...] | None = None


class ModelAdapter:
    name = "base"

    @classmethod
    def matches(cls, arch) -> bool:
        return False

    def __init__(self, arch):
        self.arch = arch

    def runtime_policy(self, runtime_config) -> RuntimeModelPolicy:
        return RuntimeModelPolicy()

    def detect(self, model) -> ModelCapabilities:
        return ModelCapabilities(supports_lora=getattr(model, "supports_lora", False),
                                 supports_multimodal=getattr(model, "supports_multimodal", False),
                                 supports_cuda_graph=getattr(model, "supports_cuda_graph", True))

    def install_tuning_config(self, runtime_config, inference_config) -> None:
        pol = self.runtime_policy(runtime_config)
        inference_config.model_policy.update(pol.model_policy)
        inference_config.kernel_policy.update(pol.kernel_policy)

    def validate_request(self, sampling_params, prompt_len: int, lora_request=None, multi_modal_data=None) -> None:
        return None

    def build_executors(self, engine) -> Any | None:
        """Return CustomRuntimeComponents to replace the generic executors, or None."""
        return None
