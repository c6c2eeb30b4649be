"""Mutable per-engine inference settings handed to model layers with every batch
(reference: vllm/engine/inference_config.py:5-43, where it rides in ``attn_metadata["config"]``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass
class LiteInferenceConfig:
    kv_cache_dtype: str = "auto"
    k_scale: float = 1.0
    v_scale: float = 1.0
    block_size: int = 16
    fusion_level: int = 2
    model_policy: dict[str, Any] = field(default_factory=dict)
    kernel_policy: dict[str, Any] = field(default_factory=dict)
    profile_spans: bool = False
    nvtx: bool = False
    # selective (sparse) decode attention: fraction of a sequence's KV blocks that global-attention layers
    # read (0 = all of them), and how many leading blocks are always kept
    kv_select_ratio: float = 0.0
    kv_select_min_blocks: int = 4

    def model_value(self, key: str, default: Any = None) -> Any:
        return self.model_policy.get(key, default)

    def kernel_value(self, key: str, default: Any = None) -> Any:
        return self.kernel_policy.get(key, default)
