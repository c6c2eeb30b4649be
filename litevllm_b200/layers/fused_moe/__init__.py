from .fused_moe import fused_moe, fused_topk

__all__ = ["fused_moe", "fused_topk"]
