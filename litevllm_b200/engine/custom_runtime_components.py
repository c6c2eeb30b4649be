"""Components a model adapter may supply in place of the stock ones.
Reference: vllm/engine/custom_runtime_components.py:8-15."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any


@dataclass
class CustomRuntimeComponents:
    prefill_executor: Any = None
    decode_executor: Any = None
    kv_block_manager: Any = None
