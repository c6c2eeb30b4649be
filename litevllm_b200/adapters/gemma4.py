"""Gemma4 adapter: fp8-e4m3 KV cache by default (the packed-int4 KV request of the base profile maps
to fp8 for this family), sliding/global layer policy, MoE execution policy.
Reference: vllm/adapters/gemma4.py:74-285."""
from .base import ModelAdapter, ModelCapabilities, RuntimeModelPolicy


class Gemma4Adapter(ModelAdapter):
    name = "gemma4"

    @classmethod
    def matches(cls, arch) -> bool:
        return arch.family == "gemma4"

    def runtime_policy(self, runtime_config) -> RuntimeModelPolicy:
        kv = runtime_config.kv_cache_dtype
        allow_int4 = runtime_config.tuning_flag("GEMMA4_ALLOW_INT4_KV", False)
        force = "fp8" if kv in ("auto", "fp8") or (kv == "turbo_int4" and not allow_int4) else None
        if kv in ("fp16", "bf16"):
            force = None
        verified = (1,) if (not self.arch.moe.num_experts and self.arch.num_layers == 48
                            and runtime_config.tuning_flag("GEMMA4_C1_PRESET", False)) else None
        return RuntimeModelPolicy(
            force_kv_cache_dtype=force, prefill_chunk_size=1024,
            model_policy={"max_kv_heads": max(self.arch.num_kv_heads, self.arch.global_kv_heads or 0),
                          "max_head_dim": max(self.arch.head_dim, self.arch.global_head_dim or 0),
                          "moe": bool(self.arch.moe.num_experts)},
            kernel_policy={"moe_strategy": "grouped_int4"}, verified_decode_batch_sizes=verified)

    def detect(self, model) -> ModelCapabilities:
        return ModelCapabilities(supports_lora=False, supports_multimodal=getattr(model, "supports_multimodal", False))
