"""Activation modules over the native elementwise kernels (CPU tensors take the PyTorch path).
Reference: vllm/model_executor/layers/activation.py:10-43."""
from __future__ import annotations

import torch
from torch import nn

from .. import ops


def _as_2d(x: torch.Tensor):
    return x.reshape(-1, x.shape[-1]), x.shape


class Silu(nn.Module):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2, shape = _as_2d(x)
        return ops.activation(x2, "silu").view(shape)


class Gelu(nn.Module):
    """tanh approximation, as used by the Gemma family."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2, shape = _as_2d(x)
        return ops.activation(x2, "gelu_tanh").view(shape)


class SiluAndMul(nn.Module):
    """``silu(x[..., :d]) * x[..., d:]``."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2, shape = _as_2d(x)
        return ops.act_mul(x2, "silu").view(*shape[:-1], shape[-1] // 2)


class GeluAndMul(nn.Module):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2, shape = _as_2d(x)
        return ops.act_mul(x2, "gelu_tanh").view(*shape[:-1], shape[-1] // 2)


def get_act_fn(name: str) -> nn.Module:
    table = {"silu": Silu, "swish": Silu, "gelu": Gelu, "gelu_tanh": Gelu, "gelu_pytorch_tanh": Gelu}
    if name not in table:
        raise ValueError(f"unknown activation {name!r}")
    return table[name]()
