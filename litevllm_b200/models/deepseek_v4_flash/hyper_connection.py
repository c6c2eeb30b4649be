"""Manifold hyper-connections: ``hc`` residual streams per token, mixed into one layer input and
re-expanded after the layer with a doubly-stochastic (Sinkhorn) stream-mixing matrix.  Batched over
tokens.  Reference: vllm/model_executor/models/deepseek_v4_flash/hyper_connection.py:16-129."""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class HyperConnectionState:
    mixed: torch.Tensor      # [T, H]      layer input
    post: torch.Tensor       # [T, hc]     gain of the layer output per stream
    combine: torch.Tensor    # [T, hc, hc] stream-mixing matrix


def sinkhorn(scores: torch.Tensor, iterations: int = 20, eps: float = 1e-6) -> torch.Tensor:
    """``[..., n, n]`` scores -> approximately doubly-stochastic matrices."""
    out = torch.softmax(scores.float(), dim=-1) + eps
    out = out / (out.sum(dim=-2, keepdim=True) + eps)
    for _ in range(1, iterations):
        out = out / (out.sum(dim=-1, keepdim=True) + eps)
        out = out / (out.sum(dim=-2, keepdim=True) + eps)
    return out


def hyper_connection_pre(streams: torch.Tensor, fn_weight: torch.Tensor, base: torch.Tensor, scale: torch.Tensor,
                         sinkhorn_iterations: int = 20, eps: float = 1e-6) -> HyperConnectionState:
    """streams ``[T, hc, H]``; ``fn_weight`` ``[hc*H, 2*hc + hc*hc]`` (or transposed); ``base``
    ``[2*hc + hc*hc]``; ``scale`` ``[3]`` (pre, post, combine)."""
    T, hc, H = streams.shape
    n_mix = 2 * hc + hc * hc
    w = fn_weight.float()
    if w.shape == (n_mix, hc * H):
        w = w.t()
    if w.shape != (hc * H, n_mix):
        raise ValueError(f"fn_weight must be [{hc * H}, {n_mix}] or its transpose, got {tuple(fn_weight.shape)}")
    flat = streams.reshape(T, hc * H).float()
    mixes = (flat @ w) * torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + eps)
    gains = torch.cat([scale[0:1].expand(hc), scale[1:2].expand(hc), scale[2:3].expand(hc * hc)]).float()
    mixes = mixes * gains + base.float()
    pre = torch.sigmoid(mixes[:, :hc]) + eps
    post = 2.0 * torch.sigmoid(mixes[:, hc:2 * hc])
    combine = sinkhorn(mixes[:, 2 * hc:].reshape(T, hc, hc), sinkhorn_iterations, eps)
    mixed = (pre.unsqueeze(-1) * streams.float()).sum(1)
    return HyperConnectionState(mixed, post, combine)


def hyper_connection_post(output: torch.Tensor, residual_streams: torch.Tensor, state: HyperConnectionState):
    """output ``[T, H]``, residual_streams ``[T, hc, H]`` -> new streams ``[T, hc, H]``."""
    mixed = torch.einsum("tij,tih->tjh", state.combine.float(), residual_streams.float())
    return state.post.unsqueeze(-1) * output.float().unsqueeze(1) + mixed
