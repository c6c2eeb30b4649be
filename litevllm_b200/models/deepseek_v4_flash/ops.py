"""Quantisation-aware round trips of DeepSeek-V4-Flash, batched over leading dimensions.
Reference: vllm/model_executor/models/deepseek_v4_flash/ops.py:175-263 (one row at a time)."""
from __future__ import annotations

import torch

from ... import ops
from ...ops import _lib

_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def hadamard128(x: torch.Tensor) -> torch.Tensor:
    """128-point Walsh-Hadamard transform of the last dimension (natural order), scaled by 1/sqrt(128)."""
    if x.shape[-1] != 128:
        raise ValueError(f"last dimension must be 128, got {x.shape[-1]}")
    y = x.float()
    lead = y.shape[:-1]
    stride = 1
    while stride < 128:
        y = y.reshape(*lead, 128 // (2 * stride), 2, stride)
        a, b = y[..., 0, :], y[..., 1, :]
        y = torch.stack([a + b, a - b], dim=-2).reshape(*lead, 128)
        stride <<= 1
    return y * 0.08838834764831845


def _pow2_scale(amax: torch.Tensor, qmax: float) -> torch.Tensor:
    return torch.exp2(torch.ceil(torch.log2(amax / qmax)))


def e2m1_roundtrip(x: torch.Tensor, block: int = 32) -> torch.Tensor:
    """FP4 (E2M1) quantise-dequantise with one power-of-two scale per ``block`` values; ties go to
    the code with the even index."""
    y = x.float().reshape(*x.shape[:-1], x.shape[-1] // block, block)
    amax = y.abs().amax(-1, keepdim=True).clamp_min(7.052966104933725e-38)
    scale = _pow2_scale(amax, 6.0)
    q = (y / scale).clamp(-6.0, 6.0)
    a = q.abs()
    r = torch.zeros_like(a)
    for strict, edge, value in ((True, 0.25, 0.5), (False, 0.75, 1.0), (True, 1.25, 1.5), (False, 1.75, 2.0),
                                (True, 2.5, 3.0), (False, 3.5, 4.0), (True, 5.0, 6.0)):
        r = torch.where(a > edge if strict else a >= edge, torch.full_like(a, value), r)
    out = torch.where(q < 0, -1.0, 1.0) * r * scale
    return out.reshape(x.shape)


def indexer_qat(rows: torch.Tensor) -> torch.Tensor:
    """Hadamard-128 then the FP4 round trip (block 32) for indexer rows ``[..., 128]``; a CUDA fp32
    tensor runs the native kernel."""
    if rows.is_cuda:
        out = rows.float().contiguous().clone().view(-1, 128)
        _lib.check(_lib.kernels().fi_dsv4_indexer_qat(ops._p(out), out.shape[0], ops._stream()), "fi_dsv4_indexer_qat")
        return out.view(rows.shape)
    return e2m1_roundtrip(hadamard128(rows), 32)


def fp8_kv_qat(row: torch.Tensor, head_dim: int, rotary_dim: int) -> torch.Tensor:
    """FP8-E4M3 round trip of the non-rotary part of latent rows ``[..., head_dim]`` in blocks of 64
    with power-of-two scales; the rotary tail passes through."""
    n_nope = head_dim - rotary_dim
    if row.shape[-1] != head_dim or n_nope % 64 != 0 or n_nope < 0:
        raise ValueError("bad head_dim / rotary_dim for the fp8 KV round trip")
    out = row.float().clone()
    if n_nope == 0:
        return out
    blk = out[..., :n_nope].reshape(*row.shape[:-1], n_nope // 64, 64)
    amax = blk.abs().amax(-1, keepdim=True).clamp_min(1e-4)
    scale = _pow2_scale(amax, 448.0)
    q = (blk / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float()
    out[..., :n_nope] = (q * scale).reshape(*row.shape[:-1], n_nope)
    return out


def q8_k_roundtrip(row: torch.Tensor, block_size: int = 256) -> torch.Tensor:
    """Round trip through the Q8_K activation quantiser used in front of the routed experts."""
    if row.shape[-1] % block_size:
        raise ValueError("row length must be a multiple of the block size")
    b = row.float().reshape(-1, block_size)
    pos = b.abs().argmax(1, keepdim=True)
    smax = b.gather(1, pos)
    nz = smax.abs() > 0
    iscale = torch.where(nz, -127.0 / torch.where(nz, smax, torch.ones_like(smax)), torch.zeros_like(smax))
    q = torch.round(b * iscale).clamp(-128, 127)
    scale = torch.where(nz, 1.0 / torch.where(nz, iscale, torch.ones_like(iscale)), torch.zeros_like(iscale))
    return (q * scale).reshape(row.shape)
