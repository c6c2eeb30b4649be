"""Architecture name -> model class (lazy imports).  Reference: vllm/model_executor/models/
registry.py:9-82."""
from __future__ import annotations

import importlib

_MODELS = {
    # architecture string: (module, class)
    "LlamaForCausalLM": ("llama", "LlamaForCausalLM"),
    "MistralForCausalLM": ("llama", "LlamaForCausalLM"),
    "Qwen2ForCausalLM": ("llama", "LlamaForCausalLM"),
    "Qwen3ForCausalLM": ("llama", "LlamaForCausalLM"),
    "Qwen3_5ForCausalLM": ("qwen3_5", "Qwen35ForCausalLM"),
    "Qwen3_5ForConditionalGeneration": ("qwen3_5", "Qwen35ForCausalLM"),
    "Qwen3_5MoeForCausalLM": ("qwen3_5", "Qwen35ForCausalLM"),
    "Qwen3_5MoeForConditionalGeneration": ("qwen3_5", "Qwen35ForCausalLM"),
    "Qwen3NextForCausalLM": ("qwen3_5", "Qwen35ForCausalLM"),
    "Qwen2VLForConditionalGeneration": ("qwen2_vl", "Qwen2VLForConditionalGeneration"),
    "Gemma4ForCausalLM": ("gemma4", "Gemma4ForCausalLM"),
    "Gemma4ForConditionalGeneration": ("gemma4", "Gemma4ForCausalLM"),
    "DeepseekV3ForCausalLM": ("deepseek_mla", "DeepseekMLAForCausalLM"),
    "DeepseekV2ForCausalLM": ("deepseek_mla", "DeepseekMLAForCausalLM"),
    "DeepseekV4FlashForCausalLM": ("deepseek_v4_flash", "DeepseekV4FlashForCausalLM"),
}
_FAMILY_DEFAULT = {
    "llama": "LlamaForCausalLM", "qwen2": "Qwen2ForCausalLM", "qwen3_5": "Qwen3_5ForCausalLM",
    "qwen2_vl": "Qwen2VLForConditionalGeneration", "gemma4": "Gemma4ForCausalLM",
    "deepseek_mla": "DeepseekV3ForCausalLM", "deepseek_v4_flash": "DeepseekV4FlashForCausalLM",
}


class ModelRegistry:
    @staticmethod
    def supported_architectures() -> list[str]:
        return sorted(_MODELS)

    @staticmethod
    def resolve_model_cls(architecture: str, family: str | None = None):
        entry = _MODELS.get(architecture)
        if entry is None and family is not None:
            entry = _MODELS.get(_FAMILY_DEFAULT.get(family, ""))
        if entry is None:
            raise ValueError(f"Model architecture {architecture!r} is not supported; known: "
                             f"{', '.join(sorted(_MODELS))}")
        mod = importlib.import_module(f"litevllm_b200.models.{entry[0]}")
        return getattr(mod, entry[1])

    @staticmethod
    def register_model(architecture: str, module: str, cls_name: str) -> None:
        _MODELS[architecture] = (module, cls_name)
