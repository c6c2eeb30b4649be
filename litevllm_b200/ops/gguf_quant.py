"""GGUF block formats used by this engine: reference (de)quantisers in PyTorch and the CUDA entry
points (csrc/gguf/gguf_kernels.cu).

  Q8_0    34 B / 32 values : fp16 d, 32 x int8            value = d * q
  Q2_K    84 B / 256 values: 16 x (4-bit scale | 4-bit min), 64 B of 2-bit codes, fp16 d, fp16 dmin
                             value = d * sc * code - dmin * m   (16 sub-blocks of 16 values)
  IQ2_XXS 66 B / 256 values: fp16 d, 8 groups of 32 values: 4 grid-row bytes + a 32-bit word holding
                             4 x 7-bit sign indices and a 4-bit scale;
                             value = d * (0.5 + scale) * 0.25 * grid[row][j] * sign
  Q4_0    18 B / 32 values : fp16 d, 16 bytes: value j = low nibble of byte j, value j+16 = high
                             nibble;  value = d * (q - 8)
  Q4_K    144 B / 256 values: fp16 d, fp16 dmin, 12 bytes of 6-bit (scale, min) pairs for 8 sub-blocks
                             of 32, 128 bytes of nibbles (64 values share 32 bytes: low nibbles first);
                             value = d * sc * q - dmin * m
  Q6_K    210 B / 256 values: 128 bytes of low nibbles, 64 bytes of 2-bit high parts, 16 int8 scales,
                             fp16 d;  value = d * sc * (q - 32)
The block layouts are GGML's (reference decoders: vllm/model_executor/models/deepseek_v4_flash/
quant.py:61-453 and vllm/model_executor/layers/quantization/tensor.py:782-833).  Activations are kept
in 16/32-bit floats (no Q8_K activation round trip).
"""
from __future__ import annotations

import torch

from . import _DT, _count, _lib, _p, _stream

GGML_TYPES = {"F32": 0, "F16": 1, "Q4_0": 2, "Q8_0": 8, "Q2_K": 10, "Q4_K": 12, "Q6_K": 14, "IQ2_XXS": 16, "I32": 26,
              "BF16": 30}
TYPE_NAMES = {v: k for k, v in GGML_TYPES.items()}
# type -> (values per block, bytes per block)
BLOCK = {2: (32, 18), 8: (32, 34), 10: (256, 84), 12: (256, 144), 14: (256, 210), 16: (256, 66)}

_KSIGNS = None
_GRID = None


def _tables():
    """(ksigns uint8 [128], grid float32 [256, 8]) parsed from the C header that holds the data."""
    global _KSIGNS, _GRID
    if _GRID is None:
        import re
        from pathlib import Path
        txt = (Path(__file__).resolve().parent.parent.parent / "csrc" / "gguf" / "iq2_tables.h").read_text()
        grid_txt = txt[txt.index("kIq2xxsGrid"):txt.index("kIq2xsSigns")]
        g = [int(x, 16) for x in re.findall(r"0x([0-9a-f]{16})ULL", grid_txt)]
        s = [int(x, 16) for x in re.findall(r"0x([0-9a-f]{2})\b", txt[txt.index("kIq2xsSigns"):])]
        assert len(g) == 256 and len(s) == 128
        _GRID = torch.tensor([[(v >> (8 * j)) & 0xFF for j in range(8)] for v in g], dtype=torch.float32)
        _KSIGNS = torch.tensor(s, dtype=torch.uint8)
    return _KSIGNS, _GRID


def row_bytes(ggml_type: int, K: int) -> int:
    vals, nb = BLOCK[ggml_type]
    assert K % vals == 0, f"K={K} is not a multiple of the block size {vals}"
    return K // vals * nb


def _f16(raw: torch.Tensor) -> torch.Tensor:
    """uint8 [..., 2] little endian -> float32."""
    return raw.contiguous().view(torch.float16).float().squeeze(-1)


def dequantize(raw: torch.Tensor, ggml_type: int, K: int) -> torch.Tensor:
    """raw uint8 [rows, row_bytes] -> float32 [rows, K] (reference implementation, any device)."""
    rows = raw.shape[0]
    vals, nb = BLOCK[ggml_type]
    blk = raw.reshape(rows, K // vals, nb)
    if ggml_type == 8:
        d = _f16(blk[..., 0:2])
        q = blk[..., 2:].contiguous().view(torch.int8).float()
        return (d[..., None] * q).reshape(rows, K)
    if ggml_type == 10:
        scales, qs = blk[..., :16], blk[..., 16:80]
        d, dmin = _f16(blk[..., 80:82]), _f16(blk[..., 82:84])
        dl = d[..., None] * (scales & 0x0F).float()
        ml = dmin[..., None] * (scales >> 4).float()
        sh = torch.tensor([0, 2, 4, 6], device=raw.device, dtype=torch.uint8).view(1, 1, 1, 4, 1)
        codes = ((qs.reshape(rows, -1, 2, 1, 32) >> sh) & 3).reshape(rows, -1, 16, 16).float()
        return (dl[..., None] * codes - ml[..., None]).reshape(rows, K)
    if ggml_type == 2:
        d = _f16(blk[..., 0:2])
        qs = blk[..., 2:]
        q = torch.cat([qs & 0x0F, qs >> 4], dim=-1).float() - 8.0
        return (d[..., None] * q).reshape(rows, K)
    if ggml_type == 12:
        d, dmin = _f16(blk[..., 0:2]), _f16(blk[..., 2:4])
        sb = blk[..., 4:16].long()                                      # 12 bytes -> 8 x (6-bit scale, 6-bit min)
        sc_lo, mn_lo = sb[..., 0:4] & 63, sb[..., 4:8] & 63
        sc_hi = (sb[..., 8:12] & 0x0F) | ((sb[..., 0:4] >> 6) << 4)
        mn_hi = (sb[..., 8:12] >> 4) | ((sb[..., 4:8] >> 6) << 4)
        sc = torch.cat([sc_lo, sc_hi], dim=-1).float()                  # [.., 8]
        mn = torch.cat([mn_lo, mn_hi], dim=-1).float()
        qs = blk[..., 16:].reshape(rows, -1, 4, 32)                     # 4 chunks of 64 values share 32 bytes each
        q = torch.stack([qs & 0x0F, qs >> 4], dim=-2).reshape(rows, -1, 8, 32).float()   # sub-block = 2 * chunk + half
        y = d[..., None, None] * sc[..., None] * q - dmin[..., None, None] * mn[..., None]
        return y.reshape(rows, K)
    if ggml_type == 14:
        ql = blk[..., 0:128].reshape(rows, -1, 2, 64)                   # two halves of 128 values
        qh = blk[..., 128:192].reshape(rows, -1, 2, 32)
        sc = blk[..., 192:208].contiguous().view(torch.int8).float().reshape(rows, -1, 2, 8)
        d = _f16(blk[..., 208:210])
        lo = torch.stack([ql[..., 0:32] & 0x0F, ql[..., 32:64] & 0x0F, ql[..., 0:32] >> 4, ql[..., 32:64] >> 4], dim=-2)
        hi = torch.stack([(qh >> s_) & 3 for s_ in (0, 2, 4, 6)], dim=-2)
        q = (lo | (hi << 4)).float() - 32.0                              # [.., half, quarter, 32]
        # scale of value l in quarter qt: sc[l // 16 + 2 * qt]
        scq = sc.reshape(rows, -1, 2, 4, 2)                              # [.., half, quarter, l // 16]
        scv = scq[..., None].expand(*scq.shape, 16).reshape(rows, -1, 2, 4, 32)
        return (d[..., None, None, None] * scv * q).reshape(rows, K)
    if ggml_type == 16:
        ksigns, grid = _tables()
        ksigns, grid = ksigns.to(raw.device), grid.to(raw.device)
        d = _f16(blk[..., 0:2])
        qs = blk[..., 2:].reshape(rows, -1, 8, 8)                       # 8 groups x 8 bytes
        rows_idx = qs[..., :4].long()                                    # grid rows
        w = qs[..., 4:].long()
        word = w[..., 0] | (w[..., 1] << 8) | (w[..., 2] << 16) | (w[..., 3] << 24)
        db = d[..., None] * (0.5 + (word >> 28).float()) * 0.25
        sidx = torch.stack([(word >> (7 * l)) & 127 for l in range(4)], dim=-1)
        sbits = ksigns[sidx].long()
        bit = torch.arange(8, device=raw.device)
        sign = 1.0 - 2.0 * ((sbits[..., None] >> bit) & 1).float()       # [.., 8 groups, 4, 8]
        vals_ = grid[rows_idx] * sign
        return (db[..., None, None] * vals_).reshape(rows, K)
    raise ValueError(f"unsupported GGUF block type {ggml_type}")


def quantize_q8_0(w: torch.Tensor) -> torch.Tensor:
    """float [rows, K] -> raw uint8 [rows, K/32*34] (round to nearest, d = absmax / 127)."""
    rows, K = w.shape
    b = w.float().reshape(rows, K // 32, 32)
    d = b.abs().amax(-1) / 127.0
    q = torch.where(d[..., None] > 0, b / d[..., None].clamp_min(1e-30), torch.zeros_like(b)).round().clamp(-127, 127)
    out = torch.empty(rows, K // 32, 34, dtype=torch.uint8, device=w.device)
    out[..., :2] = d.to(torch.float16).view(torch.uint8).reshape(rows, K // 32, 2)
    out[..., 2:] = q.to(torch.int8).view(torch.uint8)
    return out.reshape(rows, -1)


def random_blocks(ggml_type: int, rows: int, K: int, seed: int, scale: float = 0.01, device="cpu") -> torch.Tensor:
    """Random but well-formed block payloads (synthetic checkpoints)."""
    g = torch.Generator(device=device).manual_seed(seed & 0x7FFFFFFF)
    vals, nb = BLOCK[ggml_type]
    nblk = K // vals
    raw = torch.randint(0, 256, (rows, nblk, nb), generator=g, device=device, dtype=torch.int16).to(torch.uint8)
    d = (torch.rand(rows, nblk, generator=g, device=device) * scale + scale * 0.1).to(torch.float16)
    dbytes = d.view(torch.uint8).reshape(rows, nblk, 2)
    if ggml_type in (2, 8):
        raw[..., 0:2] = dbytes
    elif ggml_type == 12:
        raw[..., 0:2] = (d * 0.05).to(torch.float16).view(torch.uint8).reshape(rows, nblk, 2)
        raw[..., 2:4] = (d * 0.1).to(torch.float16).view(torch.uint8).reshape(rows, nblk, 2)
    elif ggml_type == 14:
        raw[..., 208:210] = (d * 0.02).to(torch.float16).view(torch.uint8).reshape(rows, nblk, 2)
    elif ggml_type == 10:
        raw[..., 80:82] = dbytes
        raw[..., 82:84] = (d * 0.5).to(torch.float16).view(torch.uint8).reshape(rows, nblk, 2)
    elif ggml_type == 16:
        raw[..., 0:2] = dbytes
    return raw.reshape(rows, nblk * nb)


# ---------------------------------------------------------------------------- CUDA entry points
def dequantize_cuda(raw: torch.Tensor, ggml_type: int, K: int, dtype=torch.bfloat16, out=None) -> torch.Tensor:
    rows = raw.shape[0]
    if out is None:
        out = torch.empty(rows, K, dtype=dtype, device=raw.device)
    rc = _lib.kernels().fi_gguf_dequant(_p(raw), ggml_type, rows, K, raw.stride(0), _p(out), _DT[out.dtype], _stream())
    _lib.check(rc, "fi_gguf_dequant")
    _count()
    return out


def gguf_linear(x: torch.Tensor, raw: torch.Tensor, ggml_type: int, K: int, out=None, residual=None,
                out_dtype=None) -> torch.Tensor:
    """``x @ dequant(raw).T`` (+ residual).  Up to 8 rows of x go through the block-streaming GEMV,
    larger batches dequantise into a scratch matrix and use the dense tensor-core GEMM."""
    from . import linear, scratch
    N = raw.shape[0]
    if not x.is_cuda:
        y = x.float() @ dequantize(raw, ggml_type, K).t()
        if residual is not None:
            y = y + residual.float()
        y = y.to(out_dtype or x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    M = x.shape[0]
    out_dtype = out_dtype or x.dtype
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=x.device)
    if M <= 8:
        rc = _lib.kernels().fi_gguf_gemv(_p(x), x.stride(0), _p(raw), raw.stride(0), ggml_type, M, N, K, _p(out),
                                         out.stride(0), _p(residual), 1 if out.dtype == torch.float32 else 0,
                                         _DT[x.dtype], _stream())
        _lib.check(rc, "fi_gguf_gemv")
        _count()
        return out
    dense = scratch("gguf_dense", N * K * 2, x.device)[: N * K * 2].view(x.dtype).view(N, K)
    dequantize_cuda(raw, ggml_type, K, x.dtype, out=dense)
    return linear(x, dense, residual=residual, out=out, out_dtype=out_dtype, static_weight=False)
