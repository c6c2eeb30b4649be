"""Qwen3.5 adapter: longer prefill chunks (2048 / 1024), KV dtype left to the profile for the dense
model and pinned to 16-bit for the MoE variant (reference: vllm/adapters/qwen3_5.py:32-119)."""
from .base import ModelAdapter, ModelCapabilities, RuntimeModelPolicy


class Qwen35Adapter(ModelAdapter):
    name = "qwen3_5"

    @classmethod
    def matches(cls, arch) -> bool:
        return arch.family == "qwen3_5"

    def runtime_policy(self, runtime_config) -> RuntimeModelPolicy:
        moe = bool(self.arch.moe.num_experts)
        return RuntimeModelPolicy(force_kv_cache_dtype="fp16" if moe else None,
                                  prefill_chunk_size=2048 if runtime_config.max_model_len >= 2048 else 1024,
                                  model_policy={"stabilizer": not runtime_config.tuning_flag("DISABLE_RESIDUAL_STABILIZER")})

    def detect(self, model) -> ModelCapabilities:
        return ModelCapabilities(supports_lora=False, supports_multimodal=False, supports_cuda_graph=False,
                                 supports_prefix_cache=False)
