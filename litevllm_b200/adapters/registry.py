"""Adapter selection, most specific first: DeepSeek-V4-Flash -> DeepSeek -> Gemma4 -> Qwen2-VL -> Qwen3.5 -> Llama, else
an error (reference: vllm/adapters/registry.py:123-140)."""
from __future__ import annotations

import importlib

_ORDER = [("deepseek_v4_flash", "DeepSeekV4FlashAdapter"), ("deepseek", "DeepSeekAdapter"), ("gemma4", "Gemma4Adapter"), ("qwen2_vl", "Qwen2VLAdapter"),
          ("qwen3_5", "Qwen35Adapter"), ("llama", "LlamaAdapter")]


def adapter_classes():
    out = []
    for mod, cls in _ORDER:
        try:
            m = importlib.import_module(f"litevllm_b200.adapters.{mod}")
        except ModuleNotFoundError:
            continue
        out.append(getattr(m, cls))
    return out


def get_model_adapter(arch):
    for cls in adapter_classes():
        if cls.matches(arch):
            return cls(arch)
    raise ValueError(f"no model adapter for architecture {arch.architecture!r} (family {arch.family!r})")
