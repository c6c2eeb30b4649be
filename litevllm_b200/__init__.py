"""litevllm_b200: a Blackwell-native LLM inference engine with the capabilities and public API of
the litevLLM ("FastInference") project.  Public names mirror vllm/__init__.py:14-37 of the reference."""
from __future__ import annotations

from .version import __version__

_LAZY = {
    "LLM": ("litevllm_b200.entrypoints.llm", "LLM"),
    "AsyncLLM": ("litevllm_b200.engine.async_llm", "AsyncLLM"),
    "SamplingParams": ("litevllm_b200.sampling_params", "SamplingParams"),
    "StructuredOutputsParams": ("litevllm_b200.sampling_params", "StructuredOutputsParams"),
    "PoolingParams": ("litevllm_b200.pooling_params", "PoolingParams"),
    "TextPrompt": ("litevllm_b200.inputs", "TextPrompt"),
    "TokensPrompt": ("litevllm_b200.inputs", "TokensPrompt"),
    "EmbedsPrompt": ("litevllm_b200.inputs", "EmbedsPrompt"),
    "RequestOutput": ("litevllm_b200.outputs", "RequestOutput"),
    "CompletionOutput": ("litevllm_b200.outputs", "CompletionOutput"),
    "build_vllm_config": ("litevllm_b200.config.config_builder", "build_vllm_config"),
    "LoRARequest": ("litevllm_b200.engine.lora_runtime", "LoRARequest"),
}


def __getattr__(name: str):
    entry = _LAZY.get(name)
    if entry is None:
        raise AttributeError(f"module 'litevllm_b200' has no attribute {name!r}")
    import importlib
    value = getattr(importlib.import_module(entry[0]), entry[1])
    globals()[name] = value
    return value


def clear_cache() -> None:
    """Drop cached tables/scratch buffers and return unused device memory to the driver."""
    import torch

    from .layers import rope
    from . import ops
    rope.clear_cache()
    ops._scratch.clear()
    ops._retired.clear()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


__all__ = sorted(_LAZY) + ["clear_cache", "__version__"]
