"""Frozen runtime configuration: the single typed record the engine reads its policy from.

Resolution order for every knob: profile default -> ``[tuning_keyvals]`` / legacy env override ->
explicit ``build_vllm_config`` keyword.  ``FASTINFERENCE_KV_MAX_ACTIVE_REQUESTS`` and
``FASTINFERENCE_KV_MAX_MODEL_LEN`` are honoured here (the reference accepts them but never reads
them: vllm/engine/runtime_config.py:92-94,113-114).
"""
from __future__ import annotations

import os
from collections.abc import Mapping
from dataclasses import dataclass, field, replace

from .env_registry import collect_legacy_tuning_env, truthy
from .runtime_policy import BackendRuntimePolicy, SchedulerRuntimePolicy
from .runtime_profile import RuntimeProfile, RuntimeProfileRegistry

P = "FASTINFERENCE_"


@dataclass(frozen=True)
class RuntimeConfig:
    model_path: str
    tokenizer_path: str
    dtype: str
    max_model_len: int
    max_num_seqs: int
    max_num_batched_tokens: int
    block_size: int
    kv_cache_dtype: str
    kv_max_model_len: int | None
    kv_max_active_requests: int
    kv_max_active_requests_explicit: bool
    fusion_level: int
    policy_mode: str
    enable_decode_priority: bool
    prefill_chunk_size: int
    prefill_reserved_tokens: int
    prefill_reserve_backlog: int
    prefill_catchup_ratio: float
    prefill_microbatch_size: int
    min_prefill_chunk_size: int
    max_prefill_chunk_size: int | None
    prefill_sla_ttft_ms: float
    default_min_new_tokens: int = 0
    queue_timeout_s: float = 30.0
    async_driver_min_step_interval_s: float = 0.0002
    memory_audit_topn: int = 20
    k_scale: float = 1.0
    v_scale: float = 1.0
    use_prompt_guard: bool = True
    use_legacy_sampling: bool = False
    kv_select_ratio: float = 0.0
    kv_select_min_blocks: int = 4
    tensor_parallel_size: int = 1
    expert_parallel_size: int = 1
    comm_backend: str = "fused"
    cuda_graph_decode: bool = True
    profile_nvtx: bool = False
    profile_step_events: bool = False
    heartbeat_interval_s: float = 0.5
    heartbeat_timeout_s: float = 10.0
    debug: bool = False
    tuning_env: Mapping[str, str] = field(default_factory=dict)
    scheduler_policy: SchedulerRuntimePolicy = field(default_factory=SchedulerRuntimePolicy)
    backend_policy: BackendRuntimePolicy = field(default_factory=BackendRuntimePolicy)
    profile: RuntimeProfile | None = None

    # ------------------------------------------------------------------ helpers
    def tuning(self, short_name: str, default: str | None = None) -> str | None:
        return self.tuning_env.get(P + short_name, default)

    def tuning_flag(self, short_name: str, default: bool = False) -> bool:
        raw = self.tuning_env.get(P + short_name)
        return default if raw is None else truthy(raw)

    @classmethod
    def from_vllm_config(cls, vllm_config, *, policy_mode: str = "auto",
                         environ: Mapping[str, str] | None = None) -> "RuntimeConfig":
        fi = vllm_config.fastinference_config
        env = os.environ if environ is None else environ
        tuning: dict[str, str] = {}
        if fi.legacy_env.enabled:
            tuning.update(collect_legacy_tuning_env(env, require_flag=True))
        tuning.update(fi.tuning_keyvals)

        profile = RuntimeProfileRegistry.resolve(tuning.get(P + "PROFILE", fi.profile), fi.kv_type)

        def _int(name: str, default):
            raw = tuning.get(P + name)
            return default if raw in (None, "") else int(raw)

        def _float(name: str, default):
            raw = tuning.get(P + name)
            return default if raw in (None, "") else float(raw)

        def _flag(name: str, default: bool) -> bool:
            raw = tuning.get(P + name)
            return default if raw is None else truthy(raw)

        kv_dtype = tuning.get(P + "KV_TYPE", profile.kv_cache_dtype)
        if _flag("KV_FP8", False):
            kv_dtype = "fp8"
        explicit_active = (P + "KV_MAX_ACTIVE_REQUESTS") in tuning
        backend = profile.backend_policy
        backend = replace(
            backend,
            max_prefix_cache_entries=_int("PREFIX_CACHE_MAX_ENTRIES", backend.max_prefix_cache_entries),
            max_prefix_cache_bytes=_int("PREFIX_CACHE_MAX_BYTES", backend.max_prefix_cache_bytes),
            gpu_greedy_sampling=_flag("GPU_GREEDY_SAMPLING", backend.gpu_greedy_sampling),
            gpu_greedy_max_tokens_only=_flag("GPU_GREEDY_MAX_TOKENS_ONLY", backend.gpu_greedy_max_tokens_only),
            gpu_greedy_ignore_eos=_flag("GPU_GREEDY_IGNORE_EOS", backend.gpu_greedy_ignore_eos),
            cuda_graph_decode=_flag("CUDA_GRAPH_DECODE", backend.cuda_graph_decode))
        sched = replace(profile.scheduler_policy,
                        max_decode_streak=_int("MAX_DECODE_STREAK", profile.scheduler_policy.max_decode_streak))
        mc, sc, pc = vllm_config.model_config, vllm_config.scheduler_config, vllm_config.parallel_config
        return cls(
            model_path=mc.model, tokenizer_path=mc.tokenizer, dtype=str(mc.dtype).replace("torch.", ""),
            max_model_len=mc.max_model_len, max_num_seqs=sc.max_num_seqs,
            max_num_batched_tokens=sc.max_num_batched_tokens,
            block_size=_int("BLOCK_SIZE", profile.block_size), kv_cache_dtype=kv_dtype,
            kv_max_model_len=_int("KV_MAX_MODEL_LEN", profile.kv_max_model_len),
            kv_max_active_requests=_int("KV_MAX_ACTIVE_REQUESTS", profile.kv_max_active_requests),
            kv_max_active_requests_explicit=explicit_active or profile.kv_max_active_requests != 4,
            fusion_level=_int("FUSION_LEVEL", profile.fusion_level), policy_mode=policy_mode,
            enable_decode_priority=_flag("LITE_DECODE_PRIORITY", profile.enable_decode_priority),
            prefill_chunk_size=_int("LITE_PREFILL_CHUNK", profile.prefill_chunk_size),
            prefill_reserved_tokens=_int("LITE_PREFILL_RESERVED_TOKENS", profile.prefill_reserved_tokens),
            prefill_reserve_backlog=_int("LITE_PREFILL_RESERVE_BACKLOG", profile.prefill_reserve_backlog),
            prefill_catchup_ratio=_float("LITE_PREFILL_CATCHUP_RATIO", profile.prefill_catchup_ratio),
            prefill_microbatch_size=_int("LITE_PREFILL_MICROBATCH", profile.prefill_microbatch_size),
            min_prefill_chunk_size=_int("MIN_PREFILL_CHUNK", profile.min_prefill_chunk_size),
            max_prefill_chunk_size=_int("MAX_PREFILL_CHUNK", profile.max_prefill_chunk_size),
            prefill_sla_ttft_ms=_float("SLA_TTFT_MS", profile.prefill_sla_ttft_ms),
            default_min_new_tokens=_int("LITE_DEFAULT_MIN_NEW_TOKENS", profile.default_min_new_tokens),
            queue_timeout_s=_float("LITE_QUEUE_TIMEOUT_SECONDS", profile.queue_timeout_s),
            async_driver_min_step_interval_s=profile.async_driver_min_step_interval_s,
            memory_audit_topn=_int("MEM_AUDIT_TOPN", profile.memory_audit_topn),
            k_scale=_float("K_SCALE", profile.k_scale), v_scale=_float("V_SCALE", profile.v_scale),
            use_prompt_guard=profile.use_prompt_guard,
            use_legacy_sampling=_flag("USE_LEGACY_SAMPLING", False),
            kv_select_ratio=_float("KV_SELECT_RATIO", 0.0), kv_select_min_blocks=_int("KV_SELECT_MIN_BLOCKS", 4),
            tensor_parallel_size=_int("TENSOR_PARALLEL_SIZE", pc.tensor_parallel_size),
            expert_parallel_size=_int("EXPERT_PARALLEL_SIZE", pc.expert_parallel_size),
            comm_backend=tuning.get(P + "COMM_BACKEND", pc.comm_backend),
            cuda_graph_decode=backend.cuda_graph_decode,
            profile_nvtx=_flag("PROFILE_NVTX", False), profile_step_events=_flag("PROFILE_STEP_EVENTS", False),
            heartbeat_interval_s=_float("HEARTBEAT_INTERVAL_S", 0.5),
            heartbeat_timeout_s=_float("HEARTBEAT_TIMEOUT_S", 10.0),
            debug=fi.debug or _flag("DEBUG", False), tuning_env=dict(tuning),
            scheduler_policy=sched, backend_policy=backend, profile=profile)
