"""Routers of DeepSeek-V4-Flash: a token-id -> experts table for the hash-routed layers and the
sqrt(softplus) top-k router with a selection bias.
Reference: vllm/model_executor/models/deepseek_v4_flash/moe.py:13-137."""
from __future__ import annotations

import torch

from ...ops import moe as moe_ops


def hash_routed_expert_ids(token_to_expert_ids: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
    """table ``[top_k, vocab]``, token ids ``[T]`` -> expert ids ``[T, top_k]`` (int32)."""
    if token_to_expert_ids.dim() != 2:
        raise ValueError("token_to_expert_ids must be [top_k, vocab]")
    if bool(((token_ids < 0) | (token_ids >= token_to_expert_ids.shape[1])).any()):
        raise ValueError("token id outside the routing table")
    ids = token_to_expert_ids[:, token_ids.long()].t().contiguous()
    if bool((ids < 0).any()):
        raise ValueError("hash-routed expert ids must be non-negative")
    return ids.to(torch.int32)


def sqrt_softplus_router(hidden: torch.Tensor, router_weight: torch.Tensor, top_k: int,
                         correction_bias: torch.Tensor | None = None, routed_scaling_factor: float = 1.5):
    """hidden ``[T, H]``, router weight ``[E, H]`` -> (ids int32 ``[T, k]``, weights fp32 ``[T, k]``):
    scores = sqrt(softplus(logits)), selection by score + bias, weights = normalised scores x scale.
    The scoring and top-k run in the native router kernel on a GPU."""
    logits = hidden.float() @ router_weight.float().t()
    return moe_ops.route(logits, top_k, mode="sqrt_softplus", bias=correction_bias, renormalize=True,
                         routed_scale=routed_scaling_factor)
