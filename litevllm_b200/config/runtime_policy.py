"""Small frozen policy records shared by the scheduler and the execution backend
(reference: vllm/engine/runtime_policy.py:7-19)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SchedulerRuntimePolicy:
    max_decode_streak: int = 4       # consecutive decode-only steps before a waiting prefill is forced
    max_prefill_deferrals: int = 2   # times one prefill may be skipped before it is forced
    max_admit_per_step: int = 4


@dataclass(frozen=True)
class BackendRuntimePolicy:
    max_prefix_cache_entries: int = 0         # 0 = prefix cache disabled
    max_prefix_cache_bytes: int = 1 << 30
    gpu_greedy_sampling: bool = False         # keep sampled tokens on the device, one D2H at the end
    gpu_greedy_max_tokens_only: bool = True
    gpu_greedy_ignore_eos: bool = False
    cuda_graph_decode: bool = True
    async_decode: bool = True                 # pipelined decode: launch step k+1 before reading step k
