"""Adapter for Llama / Mistral / Qwen2 / Qwen3 dense decoders (reference: vllm/adapters/llama.py:7-44)."""
from .base import ModelAdapter, RuntimeModelPolicy


class LlamaAdapter(ModelAdapter):
    name = "llama"

    @classmethod
    def matches(cls, arch) -> bool:
        return arch.family in ("llama", "qwen2")

    def runtime_policy(self, runtime_config) -> RuntimeModelPolicy:
        return RuntimeModelPolicy(prefill_chunk_size=2048)
