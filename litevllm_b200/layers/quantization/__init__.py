"""Quantisation registry: ``awq``, ``compressed-tensors`` and ``gguf``
(reference factory: vllm/model_executor/layers/quantization/__init__.py:12-27)."""
from __future__ import annotations


def get_quantization_config(quant_spec, hf_cfg: dict | None = None):
    method = getattr(quant_spec, "method", "none")
    if method in ("none", None):
        return None
    if method == "awq":
        from .awq import AWQConfig
        q = (hf_cfg or {}).get("quantization_config") or {}
        layout = "autoawq" if str(q.get("version", "")).lower() == "gemm" else "auto"
        return AWQConfig(bits=quant_spec.bits, group_size=quant_spec.group_size,
                         zero_point=quant_spec.zero_point, layout=layout)
    if method == "compressed-tensors":
        from .compressed_tensors import CompressedTensorsConfig
        return CompressedTensorsConfig(bits=quant_spec.bits, group_size=quant_spec.group_size,
                                       symmetric=quant_spec.symmetric)
    if method == "gguf":
        from .gguf import GGUFConfig
        return GGUFConfig()
    raise ValueError(f"unsupported quantization method {method!r}")
