"""Int4 weight-only quantisation helpers: checkpoint layouts -> runtime layout, reference
dequantisation, and the GEMM entry point.

Checkpoint layouts accepted (files are read unchanged, the repack happens once at load):
  * row-major ("reference") layout: ``qweight int32 [N, K/8]`` with nibble j of word w = column
    8w+j, ``scales [N, K/G]``, ``qzeros int32 [N, K/G/8]`` (vllm/model_executor/layers/quantization/
    tensor.py:835-860 of the reference); symmetric variant without zeros = ``(q - 8) * s``
    (compressed-tensors pack-quantized, tensor.py:863-901);
  * AutoAWQ GEMM layout: ``qweight int32 [K, N/8]`` with the [0,2,4,6,1,3,5,7] nibble interleave,
    ``scales [K/G, N]``, ``qzeros int32 [K/G, N/8]`` (detected by shape).
Runtime layout (csrc/gemm/awq_gemm.cu): ``qw int32 [N, K/8]`` with pair-friendly nibble order,
``scales [K/G, N]``, ``zeros uint8 [K/G, N]``.
"""
from __future__ import annotations

import torch

from . import _lib, reference
from . import _count, _p, _stream, status_word, _ACT, _DT  # noqa: F401  (shared helpers)

_AUTOAWQ_ORDER = [0, 2, 4, 6, 1, 3, 5, 7]
_SHIFTS = torch.arange(8, dtype=torch.int32) * 4


def unpack_nibbles(packed: torch.Tensor) -> torch.Tensor:
    """int32 [..., W] -> uint8 [..., W*8]; nibble j of a word is element 8w+j."""
    sh = _SHIFTS.to(packed.device)
    out = (packed.unsqueeze(-1) >> sh) & 0xF
    return out.reshape(*packed.shape[:-1], packed.shape[-1] * 8).to(torch.uint8)


def pack_nibbles(nib: torch.Tensor) -> torch.Tensor:
    """uint8 [..., W*8] -> int32 [..., W] (inverse of :func:`unpack_nibbles`)."""
    sh = _SHIFTS.to(nib.device).to(torch.int64)
    x = nib.reshape(*nib.shape[:-1], nib.shape[-1] // 8, 8).to(torch.int64)
    word = (x << sh).sum(-1)
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)
    return word.to(torch.int32)


def autoawq_to_rowmajor(qweight, scales, qzeros):
    """AutoAWQ GEMM layout -> (nibbles [N, K] uint8, scales [N, K/G], zeros [N, K/G] uint8)."""
    inv = torch.tensor([_AUTOAWQ_ORDER.index(i) for i in range(8)], device=qweight.device)
    def undo(p):   # [R, C/8] -> [R, C]
        n = unpack_nibbles(p).reshape(p.shape[0], p.shape[1], 8)
        return n[:, :, inv].reshape(p.shape[0], p.shape[1] * 8)
    nib = undo(qweight).t().contiguous()                 # [N, K]
    zeros = undo(qzeros).t().contiguous() if qzeros is not None else None   # [N, K/G]
    return nib, scales.t().contiguous(), zeros


def dequantize(nib: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor | None, group: int) -> torch.Tensor:
    """nib uint8 [N, K], scales [N, K/G], zeros uint8 [N, K/G] or None -> float32 [N, K]."""
    s = scales.float().repeat_interleave(group, dim=1)
    z = zeros.float().repeat_interleave(group, dim=1) if zeros is not None else 8.0
    return (nib.float() - z) * s


def to_runtime_layout(nib: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor | None, dtype: torch.dtype):
    """-> (qw int32 [N, K/8] pair-order, scales_t [K/G, N] dtype, zeros_t uint8 [K/G, N] | None)."""
    N, K = nib.shape
    x = nib.reshape(N, K // 8, 8).to(torch.int64)
    # word = sum_i col[2i] << 4i | col[2i+1] << (16 + 4i)
    word = torch.zeros(N, K // 8, dtype=torch.int64, device=nib.device)
    for i in range(4):
        word |= x[:, :, 2 * i] << (4 * i)
        word |= x[:, :, 2 * i + 1] << (16 + 4 * i)
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)
    return (word.contiguous(), scales.t().contiguous().to(dtype),
            zeros.t().contiguous() if zeros is not None else None)


class Int4Weight:
    """Runtime int4 weight of one (possibly merged) linear layer."""
    __slots__ = ("qw", "scales_t", "zeros_t", "group", "N", "K", "nib", "scales", "zeros")

    def __init__(self, nib, scales, zeros, group: int, dtype: torch.dtype, keep_reference: bool = False):
        self.N, self.K = nib.shape
        self.group = group
        if nib.is_cuda:
            self.qw, self.scales_t, self.zeros_t = to_runtime_layout(nib, scales, zeros, dtype)
            self.nib = self.scales = self.zeros = None
            if keep_reference:
                self.nib, self.scales, self.zeros = nib, scales, zeros
        else:
            self.qw = self.scales_t = self.zeros_t = None
            self.nib, self.scales, self.zeros = nib, scales, zeros

    @classmethod
    def from_runtime(cls, qw, scales_t, zeros_t, N: int, K: int, group: int) -> "Int4Weight":
        """Wrap tensors that already are in the kernel's layout (the on-disk repack cache)."""
        w = cls.__new__(cls)
        w.N, w.K, w.group = int(N), int(K), int(group)
        w.qw, w.scales_t, w.zeros_t = qw, scales_t, zeros_t
        w.nib = w.scales = w.zeros = None
        return w

    def dense(self) -> torch.Tensor:
        """float32 [N, K]; rebuilt from the runtime layout when the loading-time tensors were dropped."""
        if self.nib is not None:
            return dequantize(self.nib, self.scales, self.zeros, self.group)
        w = self.qw.to(torch.int64) & 0xFFFFFFFF
        cols = []
        for i in range(4):                       # word = sum_i col[2i] << 4i | col[2i+1] << (16 + 4i)
            cols += [(w >> (4 * i)) & 0xF, (w >> (16 + 4 * i)) & 0xF]
        nib = torch.stack(cols, dim=-1).reshape(self.N, self.K).to(torch.uint8)
        zeros = self.zeros_t.t().contiguous() if self.zeros_t is not None else None
        return dequantize(nib, self.scales_t.t().contiguous(), zeros, self.group)


def int4_linear(x: torch.Tensor, w: Int4Weight, bias=None, residual=None, act=None, gated_act=None,
                out=None, out_dtype=None, splits: int = 0, bn: int = 0) -> torch.Tensor:
    """``x @ dequant(w).T`` (+bias, +residual) or, with ``gated_act``, ``act(x Wg^T) * (x Wu^T)`` for
    a merged [gate; up] weight."""
    if not x.is_cuda:
        dense = w.dense().to(torch.float32)
        if gated_act:
            y = reference.gated_linear(x, dense, gated_act)
        else:
            y = reference.linear(x, dense, bias, residual, act, out_dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if w.qw is None:
        raise RuntimeError("int4 weight is not in the device runtime layout (was it loaded on the CPU?)")
    T, K = x.shape
    N = w.N // 2 if gated_act else w.N
    out_dtype = out_dtype or x.dtype
    if out is None:
        out = torch.empty(T, N, dtype=out_dtype, device=x.device)
    if T == 0:
        return out
    rc = _lib.kernels().fi_awq_gemm(
        _p(x), _p(w.qw), _p(w.scales_t), _p(w.zeros_t), _p(out), _p(bias), _p(residual), T, N, K, w.group,
        x.stride(0), out.stride(0), _ACT[gated_act if gated_act else act], N if gated_act else 0,
        1 if out.dtype == torch.float32 else 0, _DT[x.dtype], splits, bn, _p(status_word(x.device)), _stream())
    _lib.check(rc, "fi_awq_gemm")
    _count()
    return out
