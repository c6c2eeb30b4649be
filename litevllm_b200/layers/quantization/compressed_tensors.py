"""compressed-tensors ``pack-quantized`` int4 (symmetric, group 32 for Gemma4): tensors
``weight_packed int32 [N, K/8]``, ``weight_scale [N, K/G]``, ``weight_shape [2]``, optional
``weight_zero``; value = ``(nibble - 8) * scale``.  Reference: vllm/model_executor/layers/
quantization/compressed_tensors/compressed_tensors.py:53-158."""
from __future__ import annotations

from .awq import Int4LinearMethod


class CompressedTensorsConfig:
    name = "compressed-tensors"

    def __init__(self, bits: int = 4, group_size: int = 32, symmetric: bool = True,
                 skip_modules: tuple[str, ...] = ("lm_head", "router", "vision")):
        self.bits, self.group_size, self.symmetric = bits, group_size, symmetric
        self.skip_modules = skip_modules

    def get_method(self, layer):
        if any(s in layer.prefix for s in self.skip_modules) or not layer.prefix:
            return None
        return Int4LinearMethod(self.bits, self.group_size, zero_point=not self.symmetric)

    def __repr__(self) -> str:
        return f"CompressedTensorsConfig(bits={self.bits}, group_size={self.group_size}, symmetric={self.symmetric})"
