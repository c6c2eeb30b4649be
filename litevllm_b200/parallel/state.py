"""Process-wide parallel state: which rank this process is, the tensor/expert-parallel group and
the collective backend ("fused" in-kernel NVLink path or the NCCL baseline).

The reference has no distributed layer at all (its ``ColumnParallelLinear``/``RowParallelLinear``
are aliases of one plain linear, vllm/model_executor/layers/linear.py:7-11); this module is the
root of the multi-GPU extension.  With world size 1 every collective here is the identity.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class ParallelState:
    rank: int = 0
    world_size: int = 1
    tp_size: int = 1
    ep_size: int = 1
    local_rank: int = 0
    comm_backend: str = "nccl"
    group: object | None = None
    symm: object | None = None      # SymmetricHeap when the fused backend is up
    sequence_parallel_ok: bool = True   # cleared when the fused reduce-scatter / all-gather start-up check fails
    argmax_ok: bool = True              # cleared when the vocabulary-parallel arg-max start-up check fails
    self_test: dict | None = None       # verdicts of the start-up checks of the fused collectives, per form
    replica: int = 0                    # which tensor / expert-parallel group of the job this rank belongs to
    replicas: int = 1
    global_rank: int = 0                # rank in the whole job (``rank`` is the rank inside the group)

    @property
    def tp_rank(self) -> int:
        return self.rank % self.tp_size

    @property
    def ep_rank(self) -> int:
        return self.rank % self.ep_size


_STATE = ParallelState()


def get_state() -> ParallelState:
    return _STATE


def tp_size() -> int:
    return _STATE.tp_size


def tp_rank() -> int:
    return _STATE.tp_rank


def ep_size() -> int:
    return _STATE.ep_size


def ep_rank() -> int:
    return _STATE.ep_rank


def init_parallel(tp: int = 1, ep: int = 1, comm_backend: str = "fused", backend: str | None = None,
                  timeout_s: float = 600.0, replicas: int = 1) -> ParallelState:
    """Join the job described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (torchrun style).  With
    ``replicas`` > 1 the job holds that many tensor / expert-parallel groups of consecutive ranks; the state then
    describes this rank's own group (rank and size inside it) and every collective of this module runs on it."""
    global _STATE
    group_size = max(tp, ep)
    world = group_size * max(1, replicas)
    if group_size == 1:
        _STATE = ParallelState(comm_backend=comm_backend)
        return _STATE
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    env_world = int(os.environ.get("WORLD_SIZE", str(world)))
    if env_world != world:
        raise RuntimeError(f"WORLD_SIZE={env_world} does not match tp={tp} / ep={ep}"
                           + (f" x {replicas} replicas" if replicas > 1 else ""))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    use_cuda = torch.cuda.is_available()
    if backend is None:
        backend = "nccl" if use_cuda else "gloo"
    if use_cuda:
        torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    group, replica = dist.group.WORLD, 0
    if replicas > 1:
        replica = rank // group_size
        # every rank creates every group, in the same order (group creation is a collective of the whole job)
        for k in range(replicas):
            g = dist.new_group(list(range(k * group_size, (k + 1) * group_size)), backend=backend,
                               timeout=datetime.timedelta(seconds=timeout_s))
            if k == replica:
                group = g
    _STATE = ParallelState(rank=rank % group_size, world_size=group_size, tp_size=tp, ep_size=ep, local_rank=local_rank,
                           comm_backend=comm_backend, group=group)
    _STATE.replica, _STATE.replicas, _STATE.global_rank = replica, max(1, replicas), rank
    return _STATE


def destroy_parallel(destroy_group: bool = True) -> None:
    global _STATE
    if _STATE.symm is not None:
        try:
            _STATE.symm.close()
        except Exception:
            pass
    if destroy_group and dist.is_initialized():
        dist.destroy_process_group()
    _STATE = ParallelState()


# --------------------------------------------------------------------------- collectives (baseline)
def all_reduce(x: torch.Tensor) -> torch.Tensor:
    if _STATE.world_size > 1:
        dist.all_reduce(x, group=_STATE.group)
    return x


def all_gather_last_dim(x: torch.Tensor) -> torch.Tensor:
    """[.., n] on every rank -> [.., n * world] (rank-major)."""
    if _STATE.world_size == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(_STATE.world_size)]
    dist.all_gather(parts, x.contiguous(), group=_STATE.group)
    return torch.cat(parts, dim=-1)


def all_gather_rows(x: torch.Tensor) -> torch.Tensor:
    if _STATE.world_size == 1:
        return x
    out = torch.empty((x.shape[0] * _STATE.world_size, *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=_STATE.group)
    return out


def reduce_scatter_rows(x: torch.Tensor) -> torch.Tensor:
    if _STATE.world_size == 1:
        return x
    out = torch.empty((x.shape[0] // _STATE.world_size, *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x.contiguous(), group=_STATE.group)
    return out


def all_to_all_single(out: torch.Tensor, inp: torch.Tensor, out_splits=None, in_splits=None) -> torch.Tensor:
    if _STATE.world_size == 1:
        out.copy_(inp)
        return out
    dist.all_to_all_single(out, inp, out_splits, in_splits, group=_STATE.group)
    return out


def broadcast_object(obj, src: int = 0):
    if _STATE.world_size == 1:
        return obj
    box = [obj]
    # ``src`` names a rank of this group; the library call wants the rank in the whole job
    dist.broadcast_object_list(box, src=_STATE.global_rank - _STATE.rank + src, group=_STATE.group)
    return box[0]


def barrier() -> None:
    if _STATE.world_size > 1:
        dist.barrier(group=_STATE.group)
