"""Token dispatch / combine for expert parallelism over the library all-to-all (the baseline tier of the
communication layer; the default expert-parallel path keeps tokens replicated and sums expert outputs inside
the combine kernel).

With tokens replicated over the expert-parallel ranks, rank r takes the r-th slice of the step's tokens, sends
each (token, expert) route to the rank that owns the expert, runs its own experts on the routes it receives,
returns the results the same way, sums each token's routes with the router weights, and an all-gather puts the
slices back together so every rank again holds every token.  Sizes travel first (one all-to-all of counts), then
rows and expert ids with per-rank split sizes; the splits are read on the host, so this path runs eagerly and is
not captured in the decode graph.  ``FI_EP_ALLTOALL=1`` selects it in the MoE layers.
Reference: none (the reference has no multi-GPU path); the requirement is the dispatch / combine all-to-all of
expert-parallel serving.
"""
from __future__ import annotations

import os

import torch

from . import state as pstate

ENABLED = os.environ.get("FI_EP_ALLTOALL", "0") == "1"


def route_plan(ids: torch.Tensor, experts_per_rank: int, world: int):
    """``ids`` ``[T, K]`` global expert ids -> (order, send_counts): ``order`` lists the ``T*K`` routes grouped by
    owning rank (stable inside a rank), ``send_counts[d]`` is how many of them go to rank d."""
    flat = ids.reshape(-1).long()
    owner = torch.div(flat, experts_per_rank, rounding_mode="floor")
    order = torch.argsort(owner, stable=True)
    send_counts = torch.bincount(owner, minlength=world)[:world]
    return order, send_counts


def dispatch_combine(x_local: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, experts_per_rank: int,
                     run_experts) -> torch.Tensor:
    """``x_local`` ``[T, H]``: this rank's tokens; ``ids`` / ``weights`` ``[T, K]`` their routes.
    ``run_experts(rows [n, H], expert_ids [n]) -> [n, H]`` applies this rank's experts to the routes it was
    sent.  Returns the weighted sum over each token's routes, ``[T, H]`` in ``x_local``'s dtype."""
    W = pstate.ep_size()
    T, H = x_local.shape
    K = ids.shape[1]
    order, send_counts = route_plan(ids, experts_per_rank, W)
    recv_counts = torch.empty_like(send_counts)
    pstate.all_to_all_single(recv_counts, send_counts)
    send_splits, recv_splits = send_counts.tolist(), recv_counts.tolist()
    send_rows = x_local[torch.div(order, K, rounding_mode="floor")].contiguous()
    send_ids = ids.reshape(-1).long()[order].contiguous()
    n_in = int(sum(recv_splits))
    recv_rows = torch.empty(n_in, H, dtype=x_local.dtype, device=x_local.device)
    recv_ids = torch.empty(n_in, dtype=torch.long, device=x_local.device)
    pstate.all_to_all_single(recv_rows, send_rows, recv_splits, send_splits)
    pstate.all_to_all_single(recv_ids, send_ids, recv_splits, send_splits)
    y = run_experts(recv_rows, recv_ids) if n_in else recv_rows
    back = torch.empty_like(send_rows)
    pstate.all_to_all_single(back, y.to(x_local.dtype).contiguous(), send_splits, recv_splits)
    routes = torch.empty(T * K, H, dtype=torch.float32, device=x_local.device)
    routes[order] = back.float()
    return (routes.view(T, K, H) * weights.float().unsqueeze(-1)).sum(1).to(x_local.dtype)


def sharded_moe(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, experts_per_rank: int,
                run_experts) -> torch.Tensor:
    """The MoE block of a step whose tokens every rank holds: each rank handles its slice through
    :func:`dispatch_combine`, an all-gather rebuilds ``[T, H]`` on every rank."""
    W, r = pstate.ep_size(), pstate.ep_rank()
    T = x.shape[0]
    per = (T + W - 1) // W
    lo, hi = min(T, r * per), min(T, (r + 1) * per)
    out_local = dispatch_combine(x[lo:hi], ids[lo:hi], weights[lo:hi], experts_per_rank, run_experts)
    padded = torch.zeros(per, x.shape[1], dtype=x.dtype, device=x.device)
    padded[: hi - lo] = out_local
    return pstate.all_gather_rows(padded)[:T] if per * W != T else pstate.all_gather_rows(padded)
