"""Derives the execution plan (block size, context cap, slots, block counts, chunk sizes) and the
KV-cache plan from the runtime config, the model and the device memory.

Differences from the reference planner (vllm/engine/runtime_planner.py:56-158): the context cap of
4096 is kept as the *default* but an explicit ``kv_max_model_len`` / ``max_model_len`` can raise it;
slot count defaults to 16 on large-memory GPUs and can be raised up to ``max_num_seqs`` because a
B200 has room for far more than 16 contexts; KV capacity is still ``1 + slots * blocks_per_seq``
(every admitted request is guaranteed its whole context, no preemption).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..utils.misc import cdiv
from .kv_cache import KVLayerSpec, bytes_per_block, kv_format, kv_torch_dtype

DEFAULT_CONTEXT_CAP = 4096


@dataclass(frozen=True)
class ExecutionPlan:
    block_size: int
    max_model_len: int
    max_active_requests: int
    num_blocks_per_seq: int
    num_total_blocks: int
    step_token_budget: int
    prefill_chunk_size: int
    prefill_microbatch: int


@dataclass(frozen=True)
class KVCachePlan:
    dtype: torch.dtype
    dtype_name: str
    k_scale: float
    v_scale: float
    bytes_total: int
    fmt: int = 0          # 0 16-bit, 1 fp8 per-tensor scale, 2 fp8 row scales, 3 packed int4 row scales


class RuntimePlanner:
    def __init__(self, runtime_config, model_policy=None):
        self.rc = runtime_config
        self.model_policy = model_policy

    def build_execution_plan(self, device_total_bytes: int | None = None) -> ExecutionPlan:
        rc = self.rc
        bs = int(rc.block_size)
        max_len = min(rc.max_model_len, rc.kv_max_model_len or rc.max_model_len)
        max_len = max(bs, (max_len // bs) * bs)
        active = rc.kv_max_active_requests
        big_gpu = device_total_bytes is None or device_total_bytes > 24 * (1 << 30)
        if not rc.kv_max_active_requests_explicit and big_gpu:
            # a B200 holds far more than 16 contexts: follow the caller's max_num_seqs upward
            active = max(16, active, min(rc.max_num_seqs, 256))
        active = max(1, min(active, max(1, rc.max_num_seqs)))
        mp = self.model_policy
        if mp is not None and getattr(mp, "admission_cap", None):
            active = min(active, mp.admission_cap)
        per_seq = cdiv(max_len, bs)
        chunk = rc.prefill_chunk_size
        if chunk <= 0:
            chunk = getattr(mp, "prefill_chunk_size", 0) or (2048 if max_len >= 2048 else 1024)
        if rc.max_prefill_chunk_size:
            chunk = min(chunk, rc.max_prefill_chunk_size)
        chunk = max(rc.min_prefill_chunk_size, chunk)
        budget = max(rc.max_num_batched_tokens, active)
        return ExecutionPlan(block_size=bs, max_model_len=max_len, max_active_requests=active,
                             num_blocks_per_seq=per_seq, num_total_blocks=1 + active * per_seq,
                             step_token_budget=budget, prefill_chunk_size=chunk,
                             prefill_microbatch=max(1, rc.prefill_microbatch_size))

    def build_kv_cache_plan(self, plan: ExecutionPlan, specs: list[KVLayerSpec], model_dtype: torch.dtype,
                            forced_dtype: str | None = None) -> KVCachePlan:
        name = forced_dtype or self.rc.kv_cache_dtype
        dt = kv_torch_dtype(name, model_dtype)
        fmt = kv_format(name)
        if fmt == 3 and any(s.head_dim % 32 or s.v_dim % 32 for s in specs if s.num_kv_heads > 0):
            name, dt, fmt = "fp8", kv_torch_dtype("fp8", model_dtype), 1      # odd head widths cannot be nibble-packed
        total = bytes_per_block(specs, plan.block_size, dt, fmt) * plan.num_total_blocks
        return KVCachePlan(dtype=dt, dtype_name=name, k_scale=self.rc.k_scale, v_scale=self.rc.v_scale,
                           bytes_total=total, fmt=fmt)
