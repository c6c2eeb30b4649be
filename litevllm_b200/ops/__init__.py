"""Op layer: one Python function per hot op.

CUDA tensors go to the hand-written sm_100a kernels (``csrc/``, bound through ctypes); CPU tensors
go to the PyTorch fp32 reference in :mod:`litevllm_b200.ops.reference`, which doubles as the test
oracle.  There is no eager fallback for CUDA tensors: a missing native library raises.
"""
from __future__ import annotations

import math

import ctypes
import os

import torch

from . import _lib, reference

_ACT = {None: 0, "none": 0, "silu": 1, "gelu_tanh": 2, "gelu_pytorch_tanh": 2, "gelu": 2}
_DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}

_status_words: dict[int, torch.Tensor] = {}
_launches = [0]


# FI_BOUNDS_CHECK=1: every op that follows an index tensor (block tables, cache slots, token ids, row
# indices) first validates it against the extent of the buffer it indexes and raises an IndexError that
# names the operand, the offending value and its position.  The checks read the tensors back (one
# synchronisation per op), so this is a debugging mode: it finds the bad table entry that a memory
# checker would report as an out-of-bounds access, before the kernel is launched.
_BOUNDS_CHECK = os.environ.get("FI_BOUNDS_CHECK", "0") == "1"


def set_bounds_check(on: bool) -> None:
    global _BOUNDS_CHECK
    _BOUNDS_CHECK = bool(on)


def _check_index(name: str, idx: torch.Tensor, lo: int, hi: int, what: str) -> None:
    """Raise unless every element of ``idx`` lies in ``[lo, hi)``."""
    if idx is None or idx.numel() == 0:
        return
    bad = (idx < lo) | (idx >= hi)
    if bool(bad.any()):
        pos = torch.nonzero(bad)[0].tolist()
        val = int(idx[tuple(pos)])
        raise IndexError(f"{name}: value {val} at position {pos} is outside [{lo}, {hi}) ({what})")


def _check_paged(name: str, block_tables, seq_lens, k_cache, cu_q=None) -> None:
    num_blocks, bs = k_cache.shape[0], k_cache.shape[2]
    cap = block_tables.shape[1] * bs
    _check_index(name + ".seq_lens", seq_lens, 0, cap + 1, f"block table holds {cap} tokens per sequence")
    # only the entries a sequence's length reaches are followed by the kernels
    need = (seq_lens.to(torch.int64) + bs - 1) // bs
    cols = torch.arange(block_tables.shape[1], device=block_tables.device)
    used = cols[None, :] < need[:, None]
    ids = torch.where(used, block_tables.to(torch.int64), torch.zeros_like(block_tables, dtype=torch.int64))
    _check_index(name + ".block_tables", ids, 0, num_blocks, f"KV pool has {num_blocks} blocks")
    if cu_q is not None:
        d = cu_q[1:] - cu_q[:-1]
        _check_index(name + ".cu_q (differences)", d, 0, 1 << 30, "query offsets must not decrease")


def launch_count() -> int:
    """Number of native kernel launches issued by this process through the op layer (launches
    recorded while a CUDA graph is being captured count once; replays are counted by the caller)."""
    return _launches[0]


def _count(n: int = 1) -> None:
    _launches[0] += n

_scratch: dict[tuple, torch.Tensor] = {}


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """Handle of the current CUDA stream of the current device (the raw query: building a ``torch.cuda.Stream``
    object per native call costs several microseconds of host time)."""
    if _raw_stream is not None:
        return _raw_stream(_raw_device() if _raw_device is not None else torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _p(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 word that kernels set when a bounded wait runs out (0 = healthy)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        with torch.inference_mode(False):   # a normal tensor: it is reset in place from any context
            w = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[idx] = w
    return w


def check_status(device: torch.device) -> None:
    """Synchronising read of the status word; raises if any kernel reported a timeout."""
    code = int(status_word(device).item())
    if code != 0:
        status_word(device).zero_()
        raise RuntimeError(f"a device kernel reported status {code} (bounded wait ran out)")


_retired: list[torch.Tensor] = []


def scratch(name: str, nbytes: int, device: torch.device) -> torch.Tensor:
    """Grow-only cached byte buffer.  The pointer is stable while the buffer does not grow; when it
    has to grow it at least doubles, and the outgrown buffer is kept alive because CUDA graphs
    captured earlier still hold its address."""
    key = (name, device.index)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            _retired.append(buf)
        size = max(nbytes, 1 << 20, 2 * buf.numel() if buf is not None else 0)
        with torch.inference_mode(False):
            buf = torch.empty(size, dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


# ---------------------------------------------------------------------------- GEMM
# prefill-sized GEMMs take the persistent kernel (FI_PERSISTENT_GEMM=0 keeps the one-tile-per-CTA kernel)
_PERSISTENT_GEMM = os.environ.get("FI_PERSISTENT_GEMM", "1") != "0"
_PERSISTENT_MIN_T = int(os.environ.get("FI_PERSISTENT_MIN_T", "1024"))
# Plain (non-gated) products use it too, with 256-row tiles (FI_PERSISTENT_PLAIN=0 keeps the one-tile kernel)
_PERSISTENT_PLAIN = _PERSISTENT_GEMM and os.environ.get("FI_PERSISTENT_PLAIN", "1") != "0"


def _rms_scaled(x, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)


def linear(x, w, bias=None, residual=None, act=None, out=None, out_dtype=None, splits=0, bn=0, rms_eps=0.0,
           static_weight=True):
    """``act(x @ w.T) + bias + residual``.  x: [T, K], w: [N, K] (same 16-bit dtype).  With
    ``rms_eps > 0`` the rows of ``x`` are RMS-normalised (no weight: fold it into ``w``) inside the
    GEMM kernel.  ``static_weight=False`` is REQUIRED when ``w`` was written by a kernel earlier on
    the stream (a dequantised scratch copy, a computed matrix): the kernel otherwise starts reading
    weight tiles before its predecessor has finished."""
    if not x.is_cuda:
        if rms_eps > 0:
            x = _rms_scaled(x, rms_eps)
        y = reference.linear(x, w, bias, residual, act, out_dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    T, K = x.shape
    N = w.shape[0]
    out_dtype = out_dtype or x.dtype
    if out is None:
        # the kernels store 16-byte groups: rows of the output start on a multiple of 8 elements
        n8 = (N + 7) // 8 * 8
        out = torch.empty(T, n8, dtype=out_dtype, device=x.device)[:, :N]
    if T == 0:
        return out
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    if out.stride(0) % 8 != 0 or K % 8 != 0 or out.data_ptr() % 16 != 0:
        # shapes the tensor-core kernel does not take (a caller-provided narrow output, odd K): plain matmul
        y = x.float() @ w.float().t()
        if rms_eps > 0:
            y = _rms_scaled(x, rms_eps).float() @ w.float().t()
        if bias is not None:
            y = y + bias.float()
        if act:
            y = reference.apply_act(y, act)
        if residual is not None:
            y = y + residual.float()
        out.copy_(y)
        return out
    if residual is not None and residual.data_ptr() != out.data_ptr() and residual.stride(0) != out.stride(0):
        # the kernels index the residual with the output's row pitch
        if out.is_contiguous():
            residual = residual.contiguous()
        else:
            tmp = torch.empty_strided(out.shape, out.stride(), dtype=residual.dtype, device=out.device)
            tmp.copy_(residual)
            residual = tmp
    if rms_eps > 0:
        rc = _lib.kernels().fi_dense_gemm_rmsnorm(
            _p(x), _p(w), _p(out), _p(bias), _p(residual), T, N, K, x.stride(0), w.stride(0),
            out.stride(0), _ACT[act], 0, 1 if out.dtype == torch.float32 else 0, _DT[x.dtype], splits,
            bn, float(rms_eps), _p(status_word(x.device)), _stream())
        _lib.check(rc, "fi_dense_gemm_rmsnorm")
        _count()
        return out
    if _PERSISTENT_PLAIN and T >= _PERSISTENT_MIN_T and splits == 0 and bn == 0 and out.dtype == x.dtype and N % 8 == 0:
        # prefill-sized: persistent CTAs with two TMEM accumulators (epilogue overlaps the next main loop)
        rc = _lib.kernels().fi_dense_gemm_persistent(
            _p(x), _p(w), _p(out), _p(bias), _p(residual), T, N, K, x.stride(0), w.stride(0), out.stride(0),
            _ACT[act], 0, _DT[x.dtype], _p(status_word(x.device)), _stream())
        _lib.check(rc, "fi_dense_gemm_persistent")
        _count()
        return out
    fn = _lib.kernels().fi_dense_gemm if static_weight else _lib.kernels().fi_dense_gemm_dynw
    rc = fn(_p(x), _p(w), _p(out), _p(bias), _p(residual), T, N, K, x.stride(0), w.stride(0),
            out.stride(0), _ACT[act], 0, 1 if out.dtype == torch.float32 else 0, _DT[x.dtype], splits,
            bn, _p(status_word(x.device)), _stream())
    _lib.check(rc, "fi_dense_gemm")
    _count()
    return out


class FiRope(ctypes.Structure):
    _fields_ = [("cos_sin", ctypes.c_void_p), ("positions", ctypes.c_void_p), ("slot_mapping", ctypes.c_void_p),
                ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p), ("num_heads", ctypes.c_int),
                ("num_kv_heads", ctypes.c_int), ("head_dim", ctypes.c_int), ("block_size", ctypes.c_int)]


def qkv_rope_cache_supported(x, w, k_cache, nh, nkv, hd, rot_dim) -> bool:
    """Whether :func:`linear_rope_cache` can replace GEMM + rotary/cache kernel for these operands."""
    return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and k_cache.dtype == x.dtype and hd in (64, 128)
            and rot_dim == hd and w.shape[0] == (nh + 2 * nkv) * hd and x.shape[1] % 8 == 0)


def linear_rope_cache(x, w, bias, positions, cos_sin, slot_mapping, k_cache, v_cache, nh, nkv, hd, rms_eps=0.0,
                      out=None):
    """Merged q|k|v projection whose epilogue applies the rotary embedding to q and k and writes the
    new k / v rows into the paged cache (optionally with the RMSNorm of ``x`` fused in front).
    Returns the [T, (nh + 2 nkv) * hd] buffer holding rotated q, rotated k and v."""
    T, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(T, N, dtype=x.dtype, device=x.device)
    if T == 0:
        return out
    rope = FiRope(_p(cos_sin), _p(positions), _p(slot_mapping), _p(k_cache), _p(v_cache), nh, nkv, hd,
                  k_cache.shape[2])
    rc = _lib.kernels().fi_dense_gemm_rope(_p(x), _p(w), _p(out), _p(bias), T, N, K, x.stride(0), w.stride(0),
                                           out.stride(0), _DT[x.dtype], 0, 0, float(rms_eps), ctypes.byref(rope),
                                           _p(status_word(x.device)), _stream())
    _lib.check(rc, "fi_dense_gemm_rope")
    _count()
    return out


def gated_linear(x, w_gate_up, act="silu", out=None, splits=0, bn=0, rms_eps=0.0):
    """``act(x @ Wg.T) * (x @ Wu.T)`` with ``w_gate_up = [Wg; Wu]`` of shape [2*I, K] -> [T, I]
    (``rms_eps > 0``: rows of ``x`` RMS-normalised inside the kernel)."""
    if not x.is_cuda:
        if rms_eps > 0:
            x = _rms_scaled(x, rms_eps)
        y = reference.gated_linear(x, w_gate_up, act)
        if out is not None:
            out.copy_(y)
            return out
        return y
    T, K = x.shape
    inter = w_gate_up.shape[0] // 2
    if out is None:
        out = torch.empty(T, inter, dtype=x.dtype, device=x.device)
    if T == 0:
        return out
    if rms_eps <= 0 and _PERSISTENT_GEMM and T >= _PERSISTENT_MIN_T and splits == 0 and bn == 0 and inter % 8 == 0:
        rc = _lib.kernels().fi_dense_gemm_persistent(
            _p(x), _p(w_gate_up), _p(out), None, None, T, inter, K, x.stride(0), w_gate_up.stride(0), out.stride(0),
            _ACT[act], inter, _DT[x.dtype], _p(status_word(x.device)), _stream())
        _lib.check(rc, "fi_dense_gemm_persistent(gated)")
        _count()
        return out
    if rms_eps > 0:
        rc = _lib.kernels().fi_dense_gemm_rmsnorm(
            _p(x), _p(w_gate_up), _p(out), None, None, T, inter, K, x.stride(0), w_gate_up.stride(0),
            out.stride(0), _ACT[act], inter, 0, _DT[x.dtype], splits, bn, float(rms_eps),
            _p(status_word(x.device)), _stream())
    else:
        rc = _lib.kernels().fi_dense_gemm(
            _p(x), _p(w_gate_up), _p(out), None, None, T, inter, K, x.stride(0), w_gate_up.stride(0),
            out.stride(0), _ACT[act], inter, 0, _DT[x.dtype], splits, bn,
            _p(status_word(x.device)), _stream())
    _lib.check(rc, "fi_dense_gemm(gated)")
    _count()
    return out


# ---------------------------------------------------------------------------- norms
def rmsnorm(x, w, eps, residual=None, w_mode=0, out=None, out_scale=1.0, addend=None):
    """RMSNorm over the last dim of a 2-D tensor.  With ``residual`` the sum x+residual is written
    back into ``residual`` first (in place) and normalised.  With ``addend`` the result is
    ``norm(x) * w + addend`` (sandwich-norm residual add).  Returns ``out``."""
    if not x.is_cuda:
        y, new_res = reference.rmsnorm(x, w, eps, residual, w_mode, out_scale)
        if addend is not None:
            y = (y.float() + addend.float()).to(y.dtype)
        if residual is not None:
            residual.copy_(new_res)
        if out is not None:
            out.copy_(y)
            return out
        return y
    rows, H = x.shape
    if out is None:
        out = torch.empty_like(x)
    if residual is not None:
        assert residual.stride(0) == x.stride(0)
    rc = _lib.kernels().fi_rmsnorm(_p(x), _p(residual), _p(w), _p(out), rows, H, x.stride(0),
                                   out.stride(0), eps, w_mode, out_scale, _DT[x.dtype], _stream(), _p(addend))
    _lib.check(rc, "fi_rmsnorm")
    _count()
    return out


# ---------------------------------------------------------------------------- rope + cache
def rope_and_cache(qkv, positions, cos_sin, slot_mapping, k_cache, v_cache, nh, nkv, hd, rot_dim,
                   freq_stream=None, q_norm_w=None, k_norm_w=None, qk_norm_mode=-1, v_norm=False,
                   eps=1e-6, k_scale=1.0, v_scale=1.0):
    if not qkv.is_cuda:
        return reference.rope_and_cache(qkv, positions, cos_sin, slot_mapping, k_cache, v_cache, nh,
                                        nkv, hd, rot_dim, freq_stream, q_norm_w, k_norm_w,
                                        qk_norm_mode, v_norm, eps, k_scale, v_scale)
    if _BOUNDS_CHECK:
        _check_index("rope_and_cache.slot_mapping", slot_mapping, -(1 << 31), k_cache.shape[0] * k_cache.shape[2],
                     "flat slots of the KV pool; negative = skip")
        _check_index("rope_and_cache.positions", positions, 0, cos_sin.shape[0], "rows of the cos/sin table")
    T = qkv.shape[0]
    assert qkv.is_contiguous() and positions.dtype == torch.int32
    assert slot_mapping.dtype == torch.int32
    mode = reference.kv_mode(k_cache)
    if mode >= 2:
        # row-scaled cache: rotate / normalise in place without a cache write, then quantise the k and v rows
        rc = _lib.kernels().fi_rope_cache(
            _p(qkv), _p(positions), _p(cos_sin), _p(freq_stream), None, _p(k_cache), _p(v_cache), _p(q_norm_w),
            _p(k_norm_w), T, nh, nkv, hd, rot_dim, k_cache.shape[2], 0, 1.0, 1.0, eps, qk_norm_mode,
            1 if v_norm else 0, _DT[qkv.dtype], _stream())
        _lib.check(rc, "fi_rope_cache")
        _count()
        kv = qkv.view(T, nh + 2 * nkv, hd)
        _kv_quant_rows(kv[:, nh:nh + nkv], kv[:, nh + nkv:], slot_mapping, k_cache, v_cache, mode)
        return
    rc = _lib.kernels().fi_rope_cache(
        _p(qkv), _p(positions), _p(cos_sin), _p(freq_stream), _p(slot_mapping), _p(k_cache),
        _p(v_cache), _p(q_norm_w), _p(k_norm_w), T, nh, nkv, hd, rot_dim, k_cache.shape[2],
        1 if k_cache.dtype == torch.float8_e4m3fn else 0, k_scale, v_scale, eps, qk_norm_mode,
        1 if v_norm else 0, _DT[qkv.dtype], _stream())
    _lib.check(rc, "fi_rope_cache")
    _count()


def _kv_quant_rows(k, v, slot_mapping, k_cache, v_cache, mode: int) -> None:
    """k, v: [T, nkv, hd] views (last two dims contiguous) -> row-scaled cache (formats 2 and 3)."""
    T, nkv, hd = k.shape
    assert k.stride(2) == 1 and k.stride(1) == hd and v.stride(2) == 1 and v.stride(1) == hd
    rc = _lib.kernels().fi_kv_quant_rows(_p(k), _p(v), k.stride(0), v.stride(0), _p(slot_mapping), _p(k_cache),
                                         _p(v_cache), _p(k_cache.fi_scales), _p(v_cache.fi_scales), T, nkv, hd,
                                         k_cache.shape[2], mode, _DT[k.dtype], _stream())
    _lib.check(rc, "fi_kv_quant_rows")
    _count()


def reshape_and_cache(k, v, slot_mapping, k_cache, v_cache, k_scale=1.0, v_scale=1.0):
    """k, v: [T, nkv, hd] (last two dims contiguous)."""
    if _BOUNDS_CHECK:
        _check_index("reshape_and_cache.slot_mapping", slot_mapping, -(1 << 31), k_cache.shape[0] * k_cache.shape[2],
                     "flat slots of the KV pool; negative = skip")
    if not k.is_cuda:
        return reference.reshape_and_cache(k, v, slot_mapping, k_cache, v_cache, k_scale, v_scale)
    T, nkv, hd = k.shape
    mode = reference.kv_mode(k_cache)
    if mode >= 2:
        _kv_quant_rows(k, v, slot_mapping, k_cache, v_cache, mode)
        return
    rc = _lib.kernels().fi_reshape_and_cache(
        _p(k), _p(v), _p(slot_mapping), _p(k_cache), _p(v_cache), T, k.stride(0), v.stride(0), nkv,
        hd, k_cache.shape[2], 1 if k_cache.dtype == torch.float8_e4m3fn else 0, k_scale, v_scale,
        _DT[k.dtype], _stream())
    _lib.check(rc, "fi_reshape_and_cache")
    _count()


# ---------------------------------------------------------------------------- attention
_MERGE_TICKETS = 1 << 16
_merge_ticket_buf: dict[int, torch.Tensor] = {}


def _merge_tickets(device: torch.device) -> torch.Tensor:
    """Zero-initialised ticket words of the in-kernel decode merge (the kernel leaves them zero)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _merge_ticket_buf.get(idx)
    if t is None:
        with torch.inference_mode(False):
            t = torch.zeros(_MERGE_TICKETS, dtype=torch.int32, device=device)
        _merge_ticket_buf[idx] = t
    return t


# how split-KV partials are merged: "cluster" (the split CTAs form a thread-block cluster and merge through
# distributed shared memory: one launch, no scratch), "kernel" (separate merge launch), "ticket" (last CTA merges)
_DECODE_MERGE = os.environ.get("FI_DECODE_MERGE", "cluster")
_DECODE_SPLITS = int(os.environ.get("FI_DECODE_SPLITS", "0"))
# Prefill attention kernel: "auto" = the tcgen05 kernel (128 query rows per CTA) when the longest new
# chunk has at least _PREFILL_TC_MIN_Q tokens, else the 64-row mma.sync kernel; "on" / "off" force one.
_PREFILL_TC = os.environ.get("FI_PREFILL_TC", "auto")
_PREFILL_TC_MIN_Q = int(os.environ.get("FI_PREFILL_TC_MIN_Q", "64"))


def pick_decode_splits(B: int, nkv: int, max_kv_len: int, sm_count: int = 148) -> int:
    if _DECODE_SPLITS > 0:
        return _DECODE_SPLITS
    chunks = max(1, (max_kv_len + 63) // 64)
    ctas = max(1, B * nkv)
    want = max(1, (2 * sm_count + ctas - 1) // ctas)
    return int(max(1, min(want, chunks, 32)))


def paged_attention_decode(q, k_cache, v_cache, block_tables, seq_lens, nh, nkv, hd, sm_scale,
                           window=0, softcap=0.0, k_scale=1.0, v_scale=1.0, out=None, splits=0,
                           max_kv_len=None, cu_q=None):
    """One query token per sequence.  q: [B, >= nh*hd] with row stride q.stride(0)."""
    B = seq_lens.shape[0]
    if _BOUNDS_CHECK:
        _check_paged("paged_attention_decode", block_tables, seq_lens, k_cache)
    if not q.is_cuda:
        cu = torch.arange(B + 1, dtype=torch.int32)
        y = reference.paged_attention(q, k_cache, v_cache, block_tables, seq_lens, cu, nh, nkv, hd,
                                      sm_scale, window, softcap, k_scale, v_scale)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty(B, nh * hd, dtype=q.dtype, device=q.device)
    elif not out.is_contiguous():
        # the kernels write rows of nh * hd values back to back
        tmp = paged_attention_decode(q, k_cache, v_cache, block_tables, seq_lens, nh, nkv, hd, sm_scale, window,
                                     softcap, k_scale, v_scale, None, splits, max_kv_len, cu_q)
        out.copy_(tmp)
        return out
    if splits <= 0:
        if max_kv_len is None:
            max_kv_len = block_tables.shape[1] * k_cache.shape[2]
        eff = min(max_kv_len, window) if window and window > 0 else max_kv_len
        splits = pick_decode_splits(B, nkv, eff)
    mode = reference.kv_mode(k_cache)
    if mode >= 2:
        ws_o = ws_ml = None
        if splits > 1:
            n_o = B * nh * splits * hd
            ws = scratch("decode_ws", (n_o + B * nh * splits * 2) * 4, q.device).view(torch.float32)
            ws_o, ws_ml = ws[:n_o], ws[n_o:]
        rc = _lib.kernels().fi_paged_decode_rowscaled(
            _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(k_cache.fi_scales), _p(v_cache.fi_scales), _p(out),
            _p(block_tables), _p(seq_lens), _p(ws_o), _p(ws_ml), B, nh, nkv, hd, block_tables.shape[1],
            k_cache.shape[2], int(window or 0), sm_scale, float(softcap or 0.0), mode, splits, _DT[q.dtype], _stream())
        _lib.check(rc, "fi_paged_decode_rowscaled")
        _count(2 if splits > 1 else 1)
        return out
    if 1 < splits <= 8 and _DECODE_MERGE == "cluster" and k_cache.shape[2] % 16 == 0:
        rc = _lib.kernels().fi_paged_decode_cluster(
            _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(block_tables), _p(seq_lens), B, nh, nkv, hd,
            block_tables.shape[1], k_cache.shape[2], int(window or 0), sm_scale, float(softcap or 0.0),
            1 if k_cache.dtype == torch.float8_e4m3fn else 0, k_scale, v_scale, splits, _DT[q.dtype], _stream())
        _lib.check(rc, "fi_paged_decode_cluster")
        _count()
        return out
    ws_o = ws_ml = None
    if splits > 1:
        n_o = B * nh * splits * hd
        buf = scratch("decode_ws", (n_o + B * nh * splits * 2) * 4, q.device)
        ws = buf.view(torch.float32)
        ws_o, ws_ml = ws[:n_o], ws[n_o:]
    groups = nkv * ((nh // nkv + 15) // 16)
    kv_per_split = (max_kv_len if max_kv_len is not None else block_tables.shape[1] * k_cache.shape[2]) // splits
    if splits > 1 and (kv_per_split >= 1024 or _DECODE_MERGE == "ticket") and _DECODE_MERGE != "kernel" \
            and k_cache.shape[2] % 16 == 0 and B * groups <= _MERGE_TICKETS:
        # long splits: the last split CTA merges (one launch instead of two).  Short splits keep the
        # separate merge kernel: its launch overlaps the attention kernel's tail under programmatic
        # dependent launch, while the ticket (fence + atomic) would sit on every CTA's critical path
        # (measured 1.30 -> 1.38 ms per TinyLlama decode step at 1k context with in-kernel merging).
        rc = _lib.kernels().fi_paged_decode_merged(
            _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(block_tables), _p(seq_lens),
            _p(ws_o), _p(ws_ml), _p(_merge_tickets(q.device)), B, nh, nkv, hd, block_tables.shape[1],
            k_cache.shape[2], int(window or 0), sm_scale, float(softcap or 0.0),
            1 if k_cache.dtype == torch.float8_e4m3fn else 0, k_scale, v_scale, splits, _DT[q.dtype], _stream())
        _lib.check(rc, "fi_paged_decode_merged")
        _count()
        return out
    rc = _lib.kernels().fi_paged_decode(
        _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(block_tables), _p(seq_lens),
        _p(ws_o), _p(ws_ml), B, nh, nkv, hd, block_tables.shape[1], k_cache.shape[2], int(window or 0),
        sm_scale, float(softcap or 0.0), 1 if k_cache.dtype == torch.float8_e4m3fn else 0, k_scale,
        v_scale, splits, _DT[q.dtype], _stream())
    _lib.check(rc, "fi_paged_decode")
    _count(2 if splits > 1 else 1)
    return out


def paged_metadata_snapshot(q, k_cache, block_tables, seq_lens, cu_q=None, scope: str = "") -> dict:
    """Synchronising description of one paged-attention call's addressing, for diagnostics: shapes and strides,
    the blocks every sequence needs against the width of its block-table row, the range of block ids in use and
    which rows or ids fall outside the cache.  Raises ``IndexError`` when any do.  Small batches list every row,
    large ones only ranges.  Reference: vllm/kernels/triton/paged_attention.py:223-289."""
    if q.is_cuda:
        torch.cuda.synchronize(q.device)
    bs = int(k_cache.shape[2])
    lens = [int(v) for v in seq_lens.detach().cpu().tolist()]
    table = block_tables.detach().cpu()
    need = [(n + bs - 1) // bs for n in lens]
    width = int(table.shape[1])
    short_rows = [r for r, n in enumerate(need) if n > width]
    ids = [int(b) for r, n in enumerate(need) for b in table[r, :min(n, width)].tolist()]
    bad_ids = sorted({b for b in ids if b < 0 or b >= int(k_cache.shape[0])})
    few = len(lens) <= 8
    snap = {
        "scope": scope, "query_shape": list(q.shape), "query_strides": list(q.stride()),
        "cache_shape": list(k_cache.shape), "cache_strides": list(k_cache.stride()), "cache_dtype": str(k_cache.dtype),
        "block_size": bs, "block_table_shape": list(table.shape),
        "seq_lens": lens if few else {"count": len(lens), "min": min(lens, default=None), "max": max(lens, default=None)},
        "blocks_needed": need if few else {"min": min(need, default=None), "max": max(need, default=None)},
        "block_ids": [table[r, :min(n, width)].tolist() for r, n in enumerate(need)] if few else "omitted (more than 8 rows)",
        "block_id_range": [min(ids), max(ids)] if ids else None,
        "rows_longer_than_table": short_rows, "block_ids_outside_cache": bad_ids[:8],
    }
    if cu_q is not None:
        cu = [int(v) for v in cu_q.detach().cpu().tolist()]
        snap["new_tokens"] = [b - a for a, b in zip(cu, cu[1:])] if few else {"total": cu[-1] if cu else 0}
        over = [r for r, (a, b) in enumerate(zip(cu, cu[1:])) if b - a > lens[r]] if len(cu) == len(lens) + 1 else []
        snap["rows_with_more_new_tokens_than_length"] = over
        if over:
            short_rows = short_rows or over
    if short_rows or bad_ids:
        raise IndexError(f"paged attention metadata out of range: {snap}")
    return snap


def paged_attention_prefill(q, k_cache, v_cache, block_tables, seq_lens, cu_q, max_q_len, nh, nkv,
                            hd, sm_scale, window=0, softcap=0.0, k_scale=1.0, v_scale=1.0, out=None):
    """Varlen causal attention of new tokens against the paged cache (which already holds them)."""
    if _BOUNDS_CHECK:
        _check_paged("paged_attention_prefill", block_tables, seq_lens, k_cache, cu_q)
    if not q.is_cuda:
        y = reference.paged_attention(q, k_cache, v_cache, block_tables, seq_lens, cu_q, nh, nkv, hd,
                                      sm_scale, window, softcap, k_scale, v_scale)
        if out is not None:
            out.copy_(y)
            return out
        return y
    T = q.shape[0]
    B = seq_lens.shape[0]
    if out is None:
        out = torch.empty(T, nh * hd, dtype=q.dtype, device=q.device)
    elif not out.is_contiguous():
        tmp = paged_attention_prefill(q, k_cache, v_cache, block_tables, seq_lens, cu_q, max_q_len, nh, nkv, hd,
                                      sm_scale, window, softcap, k_scale, v_scale, None)
        out.copy_(tmp)
        return out
    mode = reference.kv_mode(k_cache)
    if mode >= 2:
        rc = _lib.kernels().fi_paged_prefill_rowscaled(
            _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(k_cache.fi_scales), _p(v_cache.fi_scales), _p(out),
            _p(block_tables), _p(seq_lens), _p(cu_q), B, int(max_q_len), nh, nkv, hd, block_tables.shape[1],
            k_cache.shape[2], int(window or 0), sm_scale, float(softcap or 0.0), mode, _DT[q.dtype], _stream())
        _lib.check(rc, "fi_paged_prefill_rowscaled")
        _count()
        return out
    if (_PREFILL_TC != "off" and hd in (64, 128) and k_cache.dtype == q.dtype and (k_cache.shape[2] in (16, 32, 64) or k_cache.shape[2] % 128 == 0)
            and k_cache.is_contiguous() and v_cache.is_contiguous()
            and (_PREFILL_TC == "on" or int(max_q_len) >= _PREFILL_TC_MIN_Q)):
        rc = _lib.kernels().fi_paged_prefill_tc(
            _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(block_tables), _p(seq_lens), _p(cu_q), B, T,
            int(max_q_len), nh, nkv, hd, k_cache.shape[0], block_tables.shape[1], k_cache.shape[2], int(window or 0),
            sm_scale, float(softcap or 0.0), _DT[q.dtype], _p(status_word(q.device)), _stream())
        if rc != -12:       # -12: outside what the tensor-core kernel covers, take the general one
            _lib.check(rc, "fi_paged_prefill_tc")
            _count()
            return out
    rc = _lib.kernels().fi_paged_prefill(
        _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(block_tables), _p(seq_lens),
        _p(cu_q), B, int(max_q_len), nh, nkv, hd, block_tables.shape[1], k_cache.shape[2],
        int(window or 0), sm_scale, float(softcap or 0.0),
        1 if k_cache.dtype == torch.float8_e4m3fn else 0, k_scale, v_scale, _DT[q.dtype], _stream())
    _lib.check(rc, "fi_paged_prefill")
    _count()
    return out


# ---------------------------------------------------------------------------- small ops
def embedding(ids, table, scale=1.0, vocab_start=0, vocab_end=None, out=None):
    if _BOUNDS_CHECK and vocab_start == 0 and vocab_end is None:
        _check_index("embedding.ids", ids, 0, table.shape[0], "rows of the embedding table")
    if not table.is_cuda:
        y = reference.embedding(ids, table, scale, vocab_start, vocab_end)
        if out is not None:
            out.copy_(y)
            return out
        return y
    T, H = ids.shape[0], table.shape[1]
    vocab_end = vocab_start + table.shape[0] if vocab_end is None else vocab_end
    if out is None:
        out = torch.empty(T, H, dtype=table.dtype, device=table.device)
    assert ids.dtype == torch.int64
    rc = _lib.kernels().fi_embedding(_p(ids), _p(table), _p(out), T, H, scale, vocab_start,
                                     vocab_end, _DT[table.dtype], _stream())
    _lib.check(rc, "fi_embedding")
    _count()
    return out


def act_mul(x, act="silu", out=None):
    if not x.is_cuda:
        return reference.act_mul(x, act)
    rows, d2 = x.shape
    if out is None:
        out = torch.empty(rows, d2 // 2, dtype=x.dtype, device=x.device)
    rc = _lib.kernels().fi_act_mul(_p(x), _p(out), rows, d2 // 2, x.stride(0), _ACT[act],
                                   _DT[x.dtype], _stream())
    _lib.check(rc, "fi_act_mul")
    _count()
    return out


def activation(x, act="silu", out=None):
    """Elementwise SiLU / tanh-GELU over a 2-D tensor."""
    if not x.is_cuda:
        return reference.apply_act(x.float(), act).to(x.dtype)
    rows, d = x.shape
    if out is None:
        out = torch.empty(rows, d, dtype=x.dtype, device=x.device)
    rc = _lib.kernels().fi_act(_p(x), _p(out), rows, d, x.stride(0), out.stride(0), _ACT[act], _DT[x.dtype], _stream())
    _lib.check(rc, "fi_act")
    _count()
    return out


def slot_mapping(positions, token_seq, block_tables, block_size, out=None):
    if not positions.is_cuda:
        return reference.slot_mapping(positions, token_seq, block_tables, block_size)
    T = positions.shape[0]
    if out is None:
        out = torch.empty(T, dtype=torch.int32, device=positions.device)
    rc = _lib.kernels().fi_slot_mapping(_p(positions), _p(token_seq), _p(block_tables),
                                        block_tables.shape[1], block_size, _p(out), T, _stream())
    _lib.check(rc, "fi_slot_mapping")
    _count()
    return out


def gather_rows_i32(table, idx, out):
    """``out[r] = table[idx[r]]`` for int32 ``table`` [n, cols], int32 ``idx`` [rows] (out-of-range
    indices are clamped): the block-table rows of a decode batch."""
    if _BOUNDS_CHECK:
        _check_index("gather_rows_i32.idx", idx, 0, table.shape[0], "rows of the table")
    if not table.is_cuda:
        out.copy_(table.index_select(0, idx.long().clamp_(0, table.shape[0] - 1)))
        return out
    assert table.dtype == torch.int32 and idx.dtype == torch.int32 and out.dtype == torch.int32
    assert table.is_contiguous() and out.is_contiguous() and idx.is_contiguous()
    rc = _lib.kernels().fi_gather_rows_i32(_p(table), _p(idx), _p(out), idx.shape[0], table.shape[1], table.shape[0],
                                           _stream())
    _lib.check(rc, "fi_gather_rows_i32")
    _count()
    return out


def select_blocks(block_tables, seq_lens, block_size: int, stride: int, min_blocks: int, out_table=None, out_len=None):
    """Compact block tables for selective (sparse) decode attention: of a sequence's ``n`` KV blocks keep
    block ``i`` when ``i % stride == 0``, ``i < min_blocks`` or ``i == n - 1``.  Returns ``(table, lens)`` of
    the input shapes: the kept ids packed to the left (rest: the null block) and the token count of the
    compacted sequence.  The paged decode kernel then runs unchanged on them.
    Reference: vllm/kernels/triton/paged_attention.py:94-120 (active-block index lists)."""
    if out_table is None:
        out_table = torch.empty_like(block_tables)
    if out_len is None:
        out_len = torch.empty_like(seq_lens)
    if not block_tables.is_cuda:
        out_table.zero_()
        for r in range(block_tables.shape[0]):
            ln = int(seq_lens[r])
            n = min((ln + block_size - 1) // block_size, block_tables.shape[1]) if ln > 0 else 0
            keep = [i for i in range(n) if i % stride == 0 or i < min_blocks or i == n - 1]
            if keep:
                out_table[r, :len(keep)] = block_tables[r, keep]
            out_len[r] = (len(keep) - 1) * block_size + (ln - (n - 1) * block_size) if n > 0 else 0
        return out_table, out_len
    assert block_tables.dtype == torch.int32 and seq_lens.dtype == torch.int32
    assert block_tables.is_contiguous() and out_table.is_contiguous()
    rc = _lib.kernels().fi_select_blocks(_p(block_tables), _p(seq_lens), _p(out_table), _p(out_len),
                                         block_tables.shape[0], block_tables.shape[1], int(block_size), int(stride),
                                         int(min_blocks), _stream())
    _lib.check(rc, "fi_select_blocks")
    _count()
    return out_table, out_len


def argmax(logits, out=None):
    if not logits.is_cuda:
        r = reference.argmax(logits)
        if out is not None:
            out.copy_(r)
            return out
        return r
    rows, V = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int64, device=logits.device)
    rc = _lib.kernels().fi_argmax(_p(logits), logits.stride(0), rows, V, _p(out),
                                  _DT[logits.dtype], _stream())
    _lib.check(rc, "fi_argmax")
    _count()
    return out


def sample(logits, temperature, top_k, top_p, min_p, uniform, out=None):
    """One token per row of fp32 ``logits`` [n, V] with per-row temperature (<= 0: arg-max), top-k
    (<= 0: off), top-p (>= 1: off), min-p (<= 0: off) and one uniform number in [0, 1) per row;
    all parameters are device tensors of length n.  Native kernel, no sort of the vocabulary."""
    n, V = logits.shape
    assert logits.is_cuda and logits.dtype == torch.float32 and logits.stride(1) == 1
    if out is None:
        out = torch.empty(n, dtype=torch.int64, device=logits.device)
    rc = _lib.kernels().fi_sample(_p(logits), logits.stride(0), n, V, _p(temperature), _p(top_k), _p(top_p), _p(min_p),
                                  _p(uniform), _p(out), _stream())
    _lib.check(rc, "fi_sample")
    _count()
    return out


def default_sm_scale(hd: int) -> float:
    return 1.0 / math.sqrt(hd)
