"""Parallel layout of one serving job on a single NVSwitch box.

The reference is single-GPU (vllm/engine/lite_engine.py:146 pins ``cuda:0``); tensor and expert
parallelism are additions of this engine.  One process drives one GPU; ``world_size`` is
``tensor_parallel_size`` for dense models and ``max(tp, ep)`` for MoE models (experts are sharded
over the same ranks that hold the attention shards).  ``data_parallel_size`` > 1 runs that many whole engines
(each a single GPU, or a tensor / expert-parallel group of consecutive ranks) and shards the requests over them
(parallel/data_parallel.py).
"""
from __future__ import annotations

import os
from dataclasses import dataclass


@dataclass(frozen=True)
class ParallelConfig:
    tensor_parallel_size: int = 1
    expert_parallel_size: int = 1
    data_parallel_size: int = 1   # whole-engine replicas; requests are sharded over them
    comm_backend: str = "fused"   # "fused": in-kernel NVLink collectives; "nccl": library collectives
    rank: int = 0
    local_rank: int = 0
    master_addr: str = "127.0.0.1"
    master_port: int = 29500

    @property
    def world_size(self) -> int:
        return max(self.tensor_parallel_size, self.expert_parallel_size)

    @property
    def is_distributed(self) -> bool:
        return self.world_size > 1

    @classmethod
    def from_env(cls, tp: int = 1, ep: int = 1, comm_backend: str = "fused", dp: int = 1) -> "ParallelConfig":
        # dp > 1 with tp / ep > 1: replicas of tensor / expert-parallel groups; WORLD_SIZE = dp * max(tp, ep), ranks
        # [k * group, (k + 1) * group) form replica k (offline generation; the servers route to single-GPU replicas)
        return cls(tensor_parallel_size=tp, expert_parallel_size=ep, data_parallel_size=dp, comm_backend=comm_backend,
                   rank=int(os.environ.get("RANK", "0")),
                   local_rank=int(os.environ.get("LOCAL_RANK", "0")),
                   master_addr=os.environ.get("MASTER_ADDR", "127.0.0.1"),
                   master_port=int(os.environ.get("MASTER_PORT", "29500")))
