"""Data parallelism: N replicas of a whole single-GPU engine, one process per GPU, requests sharded.

A model that fits one GPU and whose decode step is bound by per-kernel latency rather than by bytes
(a 1B model at batch 32 on a B200) gains nothing from sharding its matrices: every tensor-parallel
step still runs the same number of kernels and adds an NVLink crossing to some of them.  Replicas
divide the batch instead; each step of each replica carries 1/N of the sequences, nothing crosses
NVLink, and the job's token rate is the sum of the replicas'.

The replica layer sits above the engine: request ``i`` of a call belongs to replica ``i % N``; results
travel back as pickled objects over a gloo group, so every rank of ``LLM.generate`` returns the whole
list in order.  A replica can also be a tensor / expert-parallel group of consecutive ranks (``LLM(data_parallel_size=D,
tensor_parallel_size=T)`` under ``WORLD_SIZE = D * T``, offline generation): the group's ranks all run the
replica's prompts and its first rank contributes the results.

The reference is single-GPU (vllm/engine/lite_engine.py:146 pins ``cuda:0``) and has no counterpart.
"""
from __future__ import annotations

import datetime
import os
from typing import Any, Sequence

import torch
import torch.distributed as dist


class DataParallelGroup:
    def __init__(self, dp_size: int, timeout_s: float = 600.0, group_size: int = 1):
        """``group_size`` > 1: every replica is a tensor / expert-parallel group of that many consecutive ranks; all
        of its ranks run the replica's share of the prompts, its first rank speaks for it in the gather."""
        self.size = int(dp_size)
        self.group_size = max(1, int(group_size))
        self.global_rank = int(os.environ.get("RANK", "0"))
        self.rank = self.global_rank // self.group_size           # the replica this process belongs to
        self.is_leader = self.global_rank % self.group_size == 0
        self.local_rank = int(os.environ.get("LOCAL_RANK", str(self.global_rank)))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world != self.size * self.group_size:
            raise RuntimeError(f"data_parallel_size={self.size} with groups of {self.group_size} needs "
                               f"WORLD_SIZE={self.size * self.group_size} (got {world}): launch one process per GPU "
                               "with torchrun")
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        self._own_group = False
        if not dist.is_initialized():
            cuda = torch.cuda.is_available()
            if cuda:
                torch.cuda.set_device(self.local_rank)
            # objects travel over gloo; device tensors (barriers, timing reductions of a caller) over NCCL
            dist.init_process_group(backend="cpu:gloo,cuda:nccl" if cuda else "gloo", rank=self.global_rank,
                                    world_size=self.size * self.group_size,
                                    timeout=datetime.timedelta(seconds=timeout_s))
            self._own_group = True

    def my_indices(self, n: int) -> list[int]:
        return list(range(self.rank, n, self.size))

    def owner_of(self, index: int) -> int:
        return index % self.size

    def gather_in_order(self, local: Sequence[Any], n: int) -> list[Any]:
        """``local[k]`` is this replica's result for item ``rank + k * size``; returns all ``n`` results in
        item order on every rank."""
        parts: list[Any] = [None] * (self.size * self.group_size)
        dist.all_gather_object(parts, list(local) if self.is_leader else None)
        out: list[Any] = [None] * n
        for r in range(self.size):
            for k, item in enumerate(parts[r * self.group_size]):
                out[r + k * self.size] = item
        return out

    def barrier(self) -> None:
        dist.barrier()

    def shutdown(self) -> None:
        if self._own_group and dist.is_initialized() and not torch.cuda.is_available():
            dist.destroy_process_group()
