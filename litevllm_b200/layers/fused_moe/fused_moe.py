"""Generic mixture-of-experts for unquantised (16-bit) expert weights.

``fused_moe(x, w1, w2, router_logits, top_k)`` with ``w1 = [E, 2*I, H]`` (gate|up) and
``w2 = [E, H, I]``: routing runs in the native router kernel, the routes are sorted by expert, every
expert with work runs the gated tcgen05 GEMM (activation in the epilogue) and the down GEMM on its
contiguous row range, and the routing weights are applied in an fp32 scatter-add.  CPU tensors take
a plain PyTorch loop.  The int4 / GGUF expert paths of the Gemma4 and DeepSeek
models use the grouped kernels in ``ops.moe`` instead.
Reference: vllm/model_executor/layers/fused_moe/fused_moe.py:4-77 (softmax -> top-k -> sort -> per
expert ``F.linear`` loop).
"""
from __future__ import annotations

import torch

from ... import ops
from ...ops import moe as moe_ops


def fused_topk(router_logits: torch.Tensor, top_k: int, renormalize: bool = True, mode: str = "softmax"):
    """-> (weights fp32 [T, k], expert ids int32 [T, k])."""
    ids, weights = moe_ops.route(router_logits.float(), top_k, mode=mode, renormalize=renormalize)
    return weights, ids


def _torch_moe(x, w1, w2, ids, weights, act):
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    inter = w1.shape[1] // 2
    for e in ids.unique().tolist():
        tok, slot = torch.nonzero(ids == e, as_tuple=True)
        h = x[tok].float() @ w1[e].float().t()
        a = ops.reference.apply_act(h[:, :inter], act) * h[:, inter:]
        y = a.to(x.dtype).float() @ w2[e].float().t()
        out.index_add_(0, tok, y * weights[tok, slot].unsqueeze(1).float())
    return out.to(x.dtype)


def fused_moe(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, router_logits: torch.Tensor, top_k: int,
              renormalize: bool = True, act: str = "silu", routing: str = "softmax") -> torch.Tensor:
    weights, ids = fused_topk(router_logits, top_k, renormalize, routing)
    if not x.is_cuda:
        return _torch_moe(x, w1, w2, ids.long(), weights, act)
    T, H = x.shape
    E = w1.shape[0]
    flat = ids.reshape(-1).long()
    order = torch.argsort(flat, stable=True)                      # routes sorted by expert
    counts = torch.bincount(flat, minlength=E).tolist()           # host sync: this path is the generic fallback
    xs = x[order // top_k].contiguous()
    ys = torch.empty(T * top_k, H, dtype=x.dtype, device=x.device)
    row = 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        a = ops.gated_linear(xs[row:row + n], w1[e], act)
        ops.linear(a, w2[e], out=ys[row:row + n])
        row += n
    w_sorted = weights.reshape(-1)[order].unsqueeze(1).to(torch.float32)
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    out.index_add_(0, order // top_k, ys.float() * w_sorted)
    return out.to(x.dtype)
