"""Tensor-parallel linear ops.

``row_parallel_linear``: every rank holds a K-slice of the weight; the partial products must be
summed over ranks and the residual added once.
  * ``comm_backend = "fused"`` (default on GPUs): ONE kernel does GEMM + all-reduce + residual: the
    tcgen05 GEMM epilogue pushes its partial tile into every peer's receive slab over NVLink,
    flags it, waits for the peers' tiles and finishes the sum (csrc/gemm/epilogue.cuh).
  * ``comm_backend = "nccl"`` (baseline, also the CPU/gloo path): GEMM, then ``all_reduce``, then
    the residual add.
The reference has no tensor parallelism (vllm/model_executor/layers/linear.py:7-11 aliases every
parallel linear to the plain one).
"""
from __future__ import annotations

import ctypes

import torch

from .. import ops
from ..ops import _lib
from . import state as pstate

import os

_parity = [0]
# decode-sized all-reduces switch from the one-hop push (every rank stores its whole partial tile into
# every peer) to the two-hop form (partials to the chunk owner, 16-bit result back) at this world size
_TWO_SHOT_MIN_WORLD = int(os.environ.get("FI_TWO_SHOT_MIN_WORLD", "4"))


# Largest world size at which prefill-sized tiles (more than 256 tokens) go through the fused forms.
# Measured on 8 GPUs (T=4096): GEMM->reduce-scatter 112 us against 78 us for GEMM + NCCL, all-gather->GEMM
# 143 against 119, GEMM->all-reduce 327 against 117: with eight ranks every CTA talks to seven peers for
# a product of a few microseconds, and the library's ring wins.  On 2 GPUs the fused forms win (1.07-1.21x).
_FUSED_PREFILL_MAX_WORLD = int(os.environ.get("FI_FUSED_PREFILL_MAX_WORLD", "4"))


def fused_prefill_ok(world: int) -> bool:
    return world <= _FUSED_PREFILL_MAX_WORLD


def decode_allreduce_format(world: int, out_dtype: torch.dtype) -> int:
    """Transfer format of a decode-sized fused all-reduce: 2 = one hop, 3 = two hops."""
    if world >= _TWO_SHOT_MIN_WORLD and out_dtype in (torch.bfloat16, torch.float16):
        return 3
    return 2


def _fused_available(x: torch.Tensor) -> bool:
    st = pstate.get_state()
    return x.is_cuda and st.comm_backend == "fused" and st.symm is not None


def row_parallel_linear(layer, x: torch.Tensor, residual: torch.Tensor | None, out: torch.Tensor | None):
    st = pstate.get_state()
    T = x.shape[0]
    N = layer.out_features
    # shapes the tcgen05 kernels take: K in whole 64-element blocks (int4) / 8-element chunks (16-bit)
    k_ok = x.shape[1] % (64 if layer.quant_method is not None else 8) == 0 and N % 8 == 0
    if _fused_available(x) and k_ok:
        heap = st.symm
        if T > 0 and T <= 256 and heap.fits_low_latency(T, N):
            fmt = decode_allreduce_format(heap.world, x.dtype if out is None else out.dtype)
            return _fused_gemm_allreduce(layer, x, residual, out, heap, fmt)   # decode: inline epochs, no flags
        xfer16 = T > 256
        elem = 2 if xfer16 else 4
        if heap.fits_recv(T, N, elem) and T > 0 and (not xfer16 or fused_prefill_ok(heap.world)):
            return _fused_gemm_allreduce(layer, x, residual, out, heap, xfer16)
    # baseline: library collective around the local GEMM
    partial = layer._matmul(x, None, None, None, use_bias=pstate.tp_rank() == 0)   # bias enters the sum once
    pstate.all_reduce(partial)
    if residual is not None:
        partial = partial + residual
    if out is not None:
        out.copy_(partial)
        return out
    return partial


def _fused_gemm_allreduce(layer, x, residual, out, heap, xfer16: bool | int, phases: int = 0):
    T, K = x.shape
    N = layer.out_features
    if out is None:
        out = torch.empty(T, N, dtype=x.dtype, device=x.device)
    comm = heap.comm_desc(mode=1, T=T, N=N, xfer_16bit=xfer16, phases=phases)
    lib = _lib.kernels()
    dt = ops._DT[x.dtype]
    bias = layer.bias      # added after the cross-rank sum by whichever rank finishes an element, so every rank passes it
    if layer.quant_method is None:
        w = layer.weight
        rc = lib.fi_dense_gemm_comm(ops._p(x), ops._p(w), ops._p(out), ops._p(bias), ops._p(residual), T, N, K,
                                    x.stride(0), w.stride(0), out.stride(0), 0, 0, 0, dt, 0, 0,
                                    ops._p(ops.status_word(x.device)), ops._stream(), ctypes.byref(comm))
        _lib.check(rc, "fi_dense_gemm_comm")
    else:
        if layer.int4 is None:
            layer.quant_method.process_weights_after_loading(layer)
        w = layer.int4
        rc = lib.fi_awq_gemm_comm(ops._p(x), ops._p(w.qw), ops._p(w.scales_t), ops._p(w.zeros_t), ops._p(out),
                                  ops._p(bias), ops._p(residual), T, N, K, w.group, x.stride(0), out.stride(0),
                                  0, 0, 0, dt, 0, 0, ops._p(ops.status_word(x.device)), ops._stream(),
                                  ctypes.byref(comm))
        _lib.check(rc, "fi_awq_gemm_comm")
    ops._count()
    return out


# --------------------------------------------------------------------------- sequence-parallel forms
def _int4_of(w):
    """``w`` is a weight matrix or a linear layer; returns the layer's runtime int4 weight or None."""
    if isinstance(w, torch.Tensor):
        return None
    if w.quant_method is None:
        return None
    if w.int4 is None:
        w.quant_method.process_weights_after_loading(w)
    return w.int4


def _dense_of(w) -> torch.Tensor:
    return w if isinstance(w, torch.Tensor) else w.weight


def gemm_reduce_scatter(x: torch.Tensor, w, residual_shard: torch.Tensor | None,
                        rows_per_rank: int, out_shard: torch.Tensor | None = None,
                        xfer_16bit: bool = True, heap=None, phases: int = 0) -> torch.Tensor:
    """``(x @ w.T)`` summed over ranks, each rank keeping token rows
    ``[rank*rows_per_rank, (rank+1)*rows_per_rank)`` (+ its residual shard).  One fused kernel.
    ``w`` is a 16-bit weight matrix or a linear layer (16-bit or int4: the int4 GEMM has the same
    collective epilogue)."""
    if heap is None:
        heap = pstate.get_state().symm
    T, K = x.shape
    q = _int4_of(w)
    N = q.N if q is not None else _dense_of(w).shape[0]
    if out_shard is None:
        out_shard = torch.empty(rows_per_rank, N, dtype=x.dtype, device=x.device)
    comm = heap.comm_desc(mode=2, T=T, N=N, xfer_16bit=xfer_16bit, rows_per_rank=rows_per_rank, phases=phases)
    if q is not None:
        rc = _lib.kernels().fi_awq_gemm_comm(
            ops._p(x), ops._p(q.qw), ops._p(q.scales_t), ops._p(q.zeros_t), ops._p(out_shard), None,
            ops._p(residual_shard), T, N, K, q.group, x.stride(0), out_shard.stride(0), 0, 0, 0, ops._DT[x.dtype], 0, 0,
            ops._p(ops.status_word(x.device)), ops._stream(), ctypes.byref(comm))
        _lib.check(rc, "fi_awq_gemm_comm(reduce_scatter)")
        ops._count()
        return out_shard
    w = _dense_of(w)
    rc = _lib.kernels().fi_dense_gemm_comm(
        ops._p(x), ops._p(w), ops._p(out_shard), None, ops._p(residual_shard), T, N, K, x.stride(0), w.stride(0),
        out_shard.stride(0), 0, 0, 0, ops._DT[x.dtype], 0, 0, ops._p(ops.status_word(x.device)), ops._stream(),
        ctypes.byref(comm))
    _lib.check(rc, "fi_dense_gemm_comm(reduce_scatter)")
    ops._count()
    return out_shard


def allgather_gemm(x_shard: torch.Tensor, w, T_total: int, rows_per_rank: int,
                   out: torch.Tensor | None = None, gated_act: str | None = None,
                   staged: bool | None = None) -> torch.Tensor:
    """``concat_over_ranks(x_shard) @ w.T`` in one kernel: every rank parks its shard in the
    symmetric token buffer; a few copier CTAs at the front of the GEMM's grid pull the peers' shards
    into a local staging matrix once (each remote byte crosses NVLink once) and flag every piece,
    while the GEMM CTAs start with the local shard and pick up the staged tiles as they land
    (``staged=True``, the default when the token count is ``world * rows_per_rank``).  With
    ``staged=False`` every CTA's TMA producer reads its token tiles straight from the owner's
    memory instead (plain, non-multicast TMA loads over NVLink): simpler, but a remote tile is
    re-read once per weight tile.  ``w`` is a 16-bit weight matrix or a linear layer; an int4 layer
    runs the int4 GEMM, whose producer pulls the token tiles from the owners (the unstaged form)."""
    st = pstate.get_state()
    heap = st.symm
    K = x_shard.shape[1]
    parity = _parity[0] & 1
    _parity[0] += 1
    buf = heap.xbuf(parity, rows_per_rank, K, x_shard.dtype)
    buf[: x_shard.shape[0]].copy_(x_shard)
    q = _int4_of(w)
    rows_w = q.N if q is not None else _dense_of(w).shape[0]
    inter = rows_w // 2 if gated_act else 0
    N = inter if gated_act else rows_w
    if out is None:
        out = torch.empty(T_total, N, dtype=x_shard.dtype, device=x_shard.device)
    if q is not None:
        comm = heap.comm_desc(mode=0, T=T_total, N=N, xfer_16bit=False, ag_world=st.world_size,
                              ag_rows_per_rank=rows_per_rank, x_parity=parity, staged=False)
        rc = _lib.kernels().fi_awq_gemm_comm(
            ops._p(buf), ops._p(q.qw), ops._p(q.scales_t), ops._p(q.zeros_t), ops._p(out), None, None, T_total, N, K,
            q.group, buf.stride(0), out.stride(0), ops._ACT[gated_act] if gated_act else 0, inter, 0,
            ops._DT[x_shard.dtype], 0, 0, ops._p(ops.status_word(x_shard.device)), ops._stream(), ctypes.byref(comm))
        _lib.check(rc, "fi_awq_gemm_comm(all_gather)")
        ops._count()
        return out
    w = _dense_of(w)
    if staged is None:
        staged = T_total == st.world_size * rows_per_rank
    comm = heap.comm_desc(mode=0, T=T_total, N=N, xfer_16bit=False, ag_world=st.world_size,
                          ag_rows_per_rank=rows_per_rank, x_parity=parity, staged=staged)
    rc = _lib.kernels().fi_dense_gemm_comm(
        ops._p(buf), ops._p(w), ops._p(out), None, None, T_total, N, K, buf.stride(0), w.stride(0), out.stride(0),
        ops._ACT[gated_act] if gated_act else 0, inter, 0, ops._DT[x_shard.dtype], 0, 0,
        ops._p(ops.status_word(x_shard.device)), ops._stream(), ctypes.byref(comm))
    _lib.check(rc, "fi_dense_gemm_comm(all_gather)")
    ops._count()
    return out


def argmax_vocab_parallel(logits_local: torch.Tensor, vocab_offset: int, out: torch.Tensor | None = None,
                          heap=None, phases: int = 0) -> torch.Tensor:
    """Greedy token of every row from vocabulary-sharded fp32 logits ``[rows, V_local]`` in one kernel:
    local arg-max, one 16-byte word per row to every peer, pick the best of ``world`` candidates (ties
    to the lowest global index).  Every rank returns the same ids."""
    if heap is None:
        heap = pstate.get_state().symm
    rows, V = logits_local.shape
    assert logits_local.dtype == torch.float32 and logits_local.stride(1) == 1
    if out is None:
        out = torch.empty(rows, dtype=torch.int64, device=logits_local.device)
    comm = heap.argmax_desc(phases)
    rc = _lib.kernels().fi_argmax_tp(ops._p(logits_local), logits_local.stride(0), rows, V, int(vocab_offset),
                                     ops._p(out), ops._p(ops.status_word(logits_local.device)), ops._stream(),
                                     ctypes.byref(comm))
    _lib.check(rc, "fi_argmax_tp")
    ops._count()
    return out


def ep_heap(x: torch.Tensor):
    """Symmetric heap to use for fused expert-parallel combines of ``x`` (None -> library collectives)."""
    st = pstate.get_state()
    return st.symm if (x.is_cuda and st.comm_backend == "fused" and st.symm is not None) else None


def all_reduce_activations(x: torch.Tensor) -> torch.Tensor:
    """Sum a replicated-layout activation over the ranks (expert-parallel combine)."""
    return pstate.all_reduce(x)
