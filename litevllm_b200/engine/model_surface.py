"""Tags a model as supported or experimental by family (reference: vllm/engine/model_surface.py:18-56)."""
from __future__ import annotations

_SUPPORTED = {"llama", "qwen2", "gemma4", "deepseek_mla"}
_EXPERIMENTAL = {"qwen3_5", "qwen2_vl"}


def resolve_model_surface(model_path: str, arch) -> dict:
    fam = arch.family
    tier = "supported" if fam in _SUPPORTED else "experimental" if fam in _EXPERIMENTAL else "unknown"
    if fam == "qwen3_5" and arch.moe.num_experts:
        tier = "experimental"
    return {"model": model_path, "family": fam, "architecture": arch.architecture, "tier": tier,
            "quantization": arch.quant.method, "moe": bool(arch.moe.num_experts)}
