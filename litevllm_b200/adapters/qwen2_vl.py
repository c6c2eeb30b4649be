"""Qwen2-VL adapter (experimental image input; reference: vllm/adapters/qwen2_vl.py)."""
from .base import ModelAdapter, ModelCapabilities, RuntimeModelPolicy


class Qwen2VLAdapter(ModelAdapter):
    name = "qwen2_vl"

    @classmethod
    def matches(cls, arch) -> bool:
        return arch.family == "qwen2_vl"

    def runtime_policy(self, runtime_config) -> RuntimeModelPolicy:
        return RuntimeModelPolicy(prefill_chunk_size=4096, model_policy={"image_input": True})

    def detect(self, model) -> ModelCapabilities:
        return ModelCapabilities(supports_lora=False, supports_multimodal=True, supports_prefix_cache=False)
