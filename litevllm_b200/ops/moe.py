"""Mixture-of-experts ops: routing and the fused expert MLP.

CUDA path (csrc/moe/moe_kernels.cu + the grouped mode of csrc/gemm/awq_gemm.cu):
  route -> align (counting sort by expert + tile table, on the device, no host sync) -> gather ->
  grouped int4 gate|up GEMM with the activation in the epilogue -> grouped int4 down GEMM ->
  weighted combine.  Only the experts in ``[e_lo, e_hi)`` (this rank's shard) are computed; with
  expert parallelism the per-rank partial outputs are summed by the caller.
CPU path: a plain per-expert loop in fp32 (the oracle).
Reference: vllm/model_executor/layers/fused_moe/fused_moe.py:4-77 (softmax/topk/sort + Python loop)
and vllm/model_executor/models/gemma4/moe.py:465-623 (execution ladder).
"""
from __future__ import annotations

import ctypes

import torch

from . import _ACT, _DT, _count, _lib, _p, _stream, reference, scratch, status_word
from .awq import Int4Weight

ROUTER_MODES = {"softmax": 0, "sigmoid": 1, "sqrt_softplus": 2}


class FiGrouped(ctypes.Structure):
    _fields_ = [("tile_expert", ctypes.c_void_p), ("tile_row0", ctypes.c_void_p), ("tile_rows", ctypes.c_void_p),
                ("n_tiles", ctypes.c_void_p), ("max_tiles", ctypes.c_int), ("num_experts", ctypes.c_int),
                ("expert_rows", ctypes.c_int), ("reserved", ctypes.c_int)]


def route(logits: torch.Tensor, top_k: int, mode: str = "softmax", bias: torch.Tensor | None = None,
          expert_scale: torch.Tensor | None = None, renormalize: bool = True, routed_scale: float = 1.0):
    """logits [T, E] float32 -> (ids int32 [T, k], weights float32 [T, k])."""
    T, E = logits.shape
    if not logits.is_cuda:
        lf = logits.float()
        if mode == "softmax":
            score = torch.softmax(lf, dim=-1)
            sel = score
        else:
            score = torch.sigmoid(lf) if mode == "sigmoid" else torch.sqrt(torch.nn.functional.softplus(lf))
            sel = score + (bias.float() if bias is not None else 0.0)
        ids = torch.topk(sel, top_k, dim=-1).indices
        w = torch.gather(score, 1, ids)
        if renormalize:
            w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
        w = w * routed_scale
        if expert_scale is not None:
            w = w * expert_scale.float()[ids]
        return ids.to(torch.int32), w.float()
    ids = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    rc = _lib.kernels().fi_moe_route(_p(logits), _p(bias), _p(expert_scale), _p(ids), _p(w), T, E, top_k,
                                     ROUTER_MODES[mode], 1 if renormalize else 0, float(routed_scale), _stream())
    _lib.check(rc, "fi_moe_route")
    _count()
    return ids, w


def _reference_experts(x, w_gate_up: Int4Weight, w_down: Int4Weight, ids, weights, num_experts, e_lo, e_hi, act):
    T, H = x.shape
    inter = w_gate_up.N // (num_experts * 2)
    gu = w_gate_up.dense().view(num_experts, 2 * inter, -1)
    dn = w_down.dense().view(num_experts, H, inter)
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    xf = x.float()
    for e in range(e_lo, e_hi):
        tok, slot = torch.nonzero(ids == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        h = xf[tok] @ gu[e - 0].t()
        a = reference.apply_act(h[:, :inter], act) * h[:, inter:]
        a = a.to(x.dtype).float()
        y = (a @ dn[e].t()).to(x.dtype).float()
        out.index_add_(0, tok, y * weights[tok, slot][:, None])
    return out.to(x.dtype)


def fused_experts(x: torch.Tensor, w_gate_up: Int4Weight, w_down: Int4Weight, ids: torch.Tensor,
                  weights: torch.Tensor, num_experts_local: int, e_lo: int, act: str = "gelu_tanh",
                  residual: torch.Tensor | None = None, ep_heap=None) -> torch.Tensor:
    """x [T, H]; stacked int4 experts (``w_gate_up``: [E_local * 2I, H], ``w_down``: [E_local * H, I]);
    ids/weights from :func:`route` (global expert ids).  Returns sum_k w * expert(x) [+ residual]
    over the local experts ``[e_lo, e_lo + num_experts_local)``.  With ``ep_heap`` (the symmetric
    heap of an expert-parallel group, GPU only) the result is also summed over the ranks."""
    T, H = x.shape
    K = ids.shape[1]
    e_hi = e_lo + num_experts_local
    inter = w_gate_up.N // (num_experts_local * 2)
    if not x.is_cuda:
        local = ids - e_lo
        out = _reference_experts(x, w_gate_up, w_down, local, weights, num_experts_local, 0, num_experts_local, act)
        return out if residual is None else (out.float() + residual.float()).to(x.dtype)
    if w_gate_up.qw is None or w_down.qw is None:
        raise RuntimeError("expert weights are not in the device runtime layout (were they loaded on the CPU?)")
    n = T * K
    bn = 16 if n // max(num_experts_local, 1) < 16 else 32 if n // num_experts_local < 48 else 64
    max_tiles = min(n, num_experts_local + (n + bn - 1) // bn)
    dev = x.device
    ints = scratch("moe_ints", (2 * n + num_experts_local + 1 + 3 * max_tiles + 8) * 4, dev).view(torch.int32)
    o = 0
    sorted_route = ints[o:o + n]; o += n
    slot_of = ints[o:o + n]; o += n
    offsets = ints[o:o + num_experts_local + 1]; o += num_experts_local + 1
    tile_expert = ints[o:o + max_tiles]; o += max_tiles
    tile_row0 = ints[o:o + max_tiles]; o += max_tiles
    tile_rows = ints[o:o + max_tiles]; o += max_tiles
    n_tiles = ints[o:o + 1]
    lib = _lib.kernels()
    st = _stream()
    rc = lib.fi_moe_align(_p(ids), n, e_lo, e_hi, bn, _p(sorted_route), _p(slot_of), _p(offsets), _p(tile_expert),
                          _p(tile_row0), _p(tile_rows), _p(n_tiles), st)
    _lib.check(rc, "fi_moe_align")
    esz = x.element_size()
    acts = scratch("moe_acts", n * (2 * H + inter) * esz + 1024, dev)
    x_sorted = acts[: n * H * esz].view(x.dtype).view(n, H)
    a_sorted = acts[n * H * esz: n * (H + inter) * esz].view(x.dtype).view(n, inter)
    y_sorted = acts[n * (H + inter) * esz: n * (2 * H + inter) * esz].view(x.dtype).view(n, H)
    rc = lib.fi_moe_gather(_p(x), _p(sorted_route), _p(offsets), num_experts_local, n, K, H, _p(x_sorted),
                           _DT[x.dtype], st)
    _lib.check(rc, "fi_moe_gather")
    g = FiGrouped(_p(tile_expert), _p(tile_row0), _p(tile_rows), _p(n_tiles), max_tiles, num_experts_local,
                  2 * inter, 0)
    sw = _p(status_word(dev))
    rc = lib.fi_awq_gemm_grouped(_p(x_sorted), _p(w_gate_up.qw), _p(w_gate_up.scales_t), _p(w_gate_up.zeros_t),
                                 _p(a_sorted), None, None, n, inter, H, w_gate_up.group, H, inter, _ACT[act], inter,
                                 0, _DT[x.dtype], 1, bn, sw, st, ctypes.byref(g))
    _lib.check(rc, "fi_awq_gemm_grouped(gate_up)")
    g2 = FiGrouped(_p(tile_expert), _p(tile_row0), _p(tile_rows), _p(n_tiles), max_tiles, num_experts_local, H, 0)
    rc = lib.fi_awq_gemm_grouped(_p(a_sorted), _p(w_down.qw), _p(w_down.scales_t), _p(w_down.zeros_t), _p(y_sorted),
                                 None, None, n, H, inter, w_down.group, inter, H, 0, 0, 0, _DT[x.dtype], 1, bn, sw,
                                 st, ctypes.byref(g2))
    _lib.check(rc, "fi_awq_gemm_grouped(down)")
    out = torch.empty(T, H, dtype=x.dtype, device=dev)
    if ep_heap is not None and ep_heap.fits_low_latency(T, H):
        # expert parallel: the combine also sums the ranks' partial outputs (one kernel, peer stores)
        comm = ep_heap.comm_desc(mode=1, T=T, N=H, xfer_16bit=2)
        rc = lib.fi_moe_combine_allreduce(_p(y_sorted), _p(slot_of), _p(weights), _p(residual), _p(out), T, K, H,
                                          _DT[x.dtype], sw, st, ctypes.byref(comm))
        _lib.check(rc, "fi_moe_combine_allreduce")
        _count(5)
        return out
    rc = lib.fi_moe_combine(_p(y_sorted), _p(slot_of), _p(weights), _p(residual), _p(out), T, K, H, _DT[x.dtype], st)
    _lib.check(rc, "fi_moe_combine")
    _count(5)
    if ep_heap is not None:       # too large for the low-latency slabs: library collective
        from ..parallel import state as pstate
        pstate.all_reduce(out)
    return out
