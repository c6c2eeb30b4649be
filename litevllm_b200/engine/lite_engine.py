"""LiteEngine: owns the model, the KV pool and the control plane of one rank.

Construction phases (reference: vllm/engine/lite_engine.py:107-411): pick the model adapter and its
runtime policy -> load the model -> detect capabilities and the load-time policy -> plan execution
and KV cache -> allocate the flat KV pool -> assemble scheduler, batch builder, executors, backend
and controller.  ``add_request`` validates and enqueues, ``step`` advances every running request by
one scheduling step, ``handle_background_error`` fails every stream and releases everything.
"""
from __future__ import annotations

import asyncio
import threading

import torch

from ..adapters.registry import get_model_adapter
from ..config.inference_config import LiteInferenceConfig
from ..layers import expert_stager
from ..config.loadtime_policy import estimate_param_bytes, select_loadtime_policy
from ..loaders import get_model, resolve_device
from ..logger import init_logger
from ..sampling_params import SamplingParams
from .errors import EngineFatalError, InvalidRequestError, RequestAbortedError, RequestRejectedError
from .initialization import LiteRuntimeAssembler, MemoryAuditor
from .observer import InMemoryRuntimeObserver
from .request_builder import LiteRequestBuilder
from .runtime_factory import LiteRuntimeFactory
from .runtime_planner import RuntimePlanner

logger = init_logger(__name__)


class LiteEngine:
    def __init__(self, vllm_config, model=None, observer=None):
        self.vllm_config = vllm_config
        self.rc = vllm_config.runtime_config
        self.model_config = vllm_config.model_config
        self.arch = self.model_config.arch
        self.device = resolve_device(vllm_config.device)
        self.observer = observer or InMemoryRuntimeObserver()
        self.tokenizer = None
        self.fatal_error: BaseException | None = None
        self.lock = threading.RLock()
        self._lazy_built = False
        self.pre_step_hook = None
        self._init_before_model_load()
        self.model = model if model is not None else get_model(vllm_config, self.device)
        self._init_after_model_load()

    # ------------------------------------------------------------------ init phases
    def _init_before_model_load(self) -> None:
        self.adapter = get_model_adapter(self.arch)
        self.model_policy = self.adapter.runtime_policy(self.rc)
        self.inf_config = LiteInferenceConfig(
            kv_cache_dtype=self.model_policy.force_kv_cache_dtype or self.rc.kv_cache_dtype,
            k_scale=self.rc.k_scale, v_scale=self.rc.v_scale, block_size=self.rc.block_size,
            fusion_level=self.rc.fusion_level, nvtx=self.rc.profile_nvtx,
            profile_spans=self.rc.profile_step_events,
            kv_select_ratio=max(0.0, min(1.0, float(self.rc.kv_select_ratio))),
            kv_select_min_blocks=max(1, int(self.rc.kv_select_min_blocks)))
        self.adapter.install_tuning_config(self.rc, self.inf_config)
        if self.inf_config.profile_spans or self.inf_config.nvtx:
            from ..utils.profiling import PROFILER
            PROFILER.configure(self.inf_config.profile_spans, self.inf_config.nvtx)

    def _device_total_bytes(self) -> int | None:
        if self.device.type == "cuda":
            return torch.cuda.get_device_properties(self.device).total_memory
        return None

    def _init_after_model_load(self) -> None:
        self.capabilities = self.adapter.detect(self.model)
        total = self._device_total_bytes()
        self.loadtime_policy = select_loadtime_policy(estimate_param_bytes(self.model), total, self.rc.policy_mode)
        planner = RuntimePlanner(self.rc, self.model_policy)
        ctx = LiteRuntimeAssembler.assemble(self, planner, total)
        self.plan, self.kv_plan = ctx.plan, ctx.kv_plan
        if total is not None:
            free, _ = torch.cuda.mem_get_info(self.device)
            budget = int(free - (1.0 - self.vllm_config.cache_config.gpu_memory_utilization) * total)
            if self.kv_plan.bytes_total > budget:
                raise MemoryError(
                    f"KV cache needs {self.kv_plan.bytes_total / 2**30:.1f} GiB for "
                    f"{self.plan.max_active_requests} x {self.plan.max_model_len} tokens but only "
                    f"{budget / 2**30:.1f} GiB are available; lower max_num_seqs or max_model_len")
        parts = LiteRuntimeFactory.build(ctx)
        for name, value in vars(parts).items():      # kv_cache, allocator, kv_manager, scheduler, builder, ...
            setattr(self, name, value)
        self.memory = MemoryAuditor().snapshot(self.model, self.kv_cache, self.device)
        logger.info("memory: %s", self.memory.report())
        from .model_surface import resolve_model_surface
        self.observer.on_model_surface(resolve_model_surface(self.model_config.model, self.arch))
        # Everything built so far (weights' Python wrappers, tokenizer tables, configs) lives as long as the
        # engine: park it in the permanent generation so the collector's full passes, which would
        # otherwise stall a decode step for tens of milliseconds now and then, have little to scan.
        import gc
        gc.collect()
        gc.freeze()
        logger.info("engine ready: %d slots x %d tokens, %d KV blocks (%s, %.2f GiB), chunk %d",
                    self.plan.max_active_requests, self.plan.max_model_len, self.plan.num_total_blocks,
                    self.kv_plan.dtype, self.kv_cache.total_bytes / 2 ** 30, self.plan.prefill_chunk_size)

    @staticmethod
    def _span_summary() -> dict:
        from ..utils.profiling import PROFILER
        return PROFILER.summary() if PROFILER.enabled else {}

    @property
    def max_active_requests(self) -> int:
        return self.plan.max_active_requests

    # ------------------------------------------------------------------ tokenizer / lazy parts
    def set_tokenizer(self, tokenizer) -> None:
        self.tokenizer = tokenizer
        self.output_pipeline.tokenizer = tokenizer
        self._lazy_built = False

    def _build_lazy(self) -> None:
        if self._lazy_built:
            return
        from .structured_output import make_constraint_factory
        cap = self.loadtime_policy.max_tokens_cap if self.loadtime_policy.name == "stable" else None
        self.request_builder = LiteRequestBuilder(
            self.tokenizer, self.plan.max_model_len, self.arch.vocab_size, self.arch.eos_token_ids, self.device,
            max_tokens_cap=cap, default_min_new_tokens=self.rc.default_min_new_tokens,
            structured_factory=make_constraint_factory(self.tokenizer, self.arch.vocab_size),
            multimodal=self.multimodal, chunked_prefill=self.capabilities.supports_chunked_prefill)
        self._lazy_built = True

    # ------------------------------------------------------------------ requests
    def add_request(self, request_id: str, prompt, sampling_params: SamplingParams | None = None,
                    lora_request=None, multi_modal_data=None, loop: asyncio.AbstractEventLoop | None = None):
        with self.lock:
            if self.fatal_error is not None:
                raise EngineFatalError(f"engine stopped after a fatal error: {self.fatal_error!r}")
            self._build_lazy()
            try:
                if lora_request is not None and self.lora_registry is None:
                    raise InvalidRequestError("this model does not support LoRA adapters")
                if multi_modal_data and self.multimodal is None:
                    raise InvalidRequestError("this model does not accept multimodal input")
                st = self.request_builder.build(request_id, prompt, sampling_params, lora_request, multi_modal_data)
                self.adapter.validate_request(st.sampling_params, st.prompt_len, lora_request, st.multi_modal_data)
                if lora_request is not None:
                    self.lora_registry.acquire(lora_request)
                self.scheduler.enqueue_request(st, loop)
            except RequestRejectedError as e:
                self.observer.on_request_rejected(request_id, e.reason)
                raise
            self.observer.on_request_added(request_id, st.prompt_len)
            return st

    def abort_request(self, request_id: str) -> bool:
        with self.lock:
            st = self.scheduler.get(request_id)
            if st is None:
                return False
            self.scheduler.publish_output(request_id, RequestAbortedError(f"request {request_id} aborted"))
            self.observer.on_request_aborted(request_id)
            self.backend.release_request(request_id)
            return True

    def _on_release(self, st) -> None:
        if st.lora_request is not None and self.lora_registry is not None:
            self.lora_registry.release(st.lora_request)

    def get_request_stream(self, request_id: str):
        return self.scheduler.get_request_stream(request_id)

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished()

    # ------------------------------------------------------------------ stepping
    @torch.inference_mode()
    def step(self) -> list:
        with self.lock:
            if self.fatal_error is not None:
                raise EngineFatalError(f"engine stopped after a fatal error: {self.fatal_error!r}")
            if self.pre_step_hook is not None:
                self.pre_step_hook()
            return self.controller.step()

    def handle_background_error(self, exc: BaseException) -> None:
        """Fatal: every stream gets the exception, every request is released, admission closes."""
        with self.lock:
            self.fatal_error = exc
            self.observer.on_background_error(exc)
            for rid in self.scheduler.all_request_ids():
                self.scheduler.publish_output(rid, exc)
                try:
                    self.backend.release_request(rid)
                except Exception:  # teardown must finish for every request
                    logger.exception("release failed for %s during fatal teardown", rid)

    # ------------------------------------------------------------------ stats / adapters
    def stats(self) -> dict:
        extra = {"profile": self.rc.profile.stats() if self.rc.profile else {},
                 "plan": self.plan.__dict__, "loadtime_policy": self.loadtime_policy.name,
                 "lora": self.lora_registry.stats() if self.lora_registry else {},
                 "multimodal": self.multimodal.stats() if self.multimodal else {},
                 "memory": self.memory.as_dict(), "profile_spans": self._span_summary(),
                 "expert_staging": expert_stager.summary(self.model),
                 "parallel": {"tp": self.rc.tensor_parallel_size, "ep": self.rc.expert_parallel_size,
                              "comm_backend": self.rc.comm_backend}}
        return self.controller.stats(extra)

    def reset_stats(self, clear_prefix_cache: bool = False) -> None:
        self.observer.reset()
        if clear_prefix_cache:
            self.prefix_cache.clear()

    def register_lora_adapter(self, lora_name: str, lora_path: str, lora_int_id: int | None = None):
        if self.lora_registry is None:
            raise InvalidRequestError("this model does not support LoRA adapters")
        return self.lora_registry.register(lora_name, lora_path, lora_int_id)

    def unregister_lora_adapter(self, lora_name: str) -> bool:
        return self.lora_registry.unregister(lora_name) if self.lora_registry else False

    def shutdown(self) -> None:
        with self.lock:
            for rid in self.scheduler.all_request_ids():
                self.abort_request(rid)
        # the engine's objects were parked in the collector's permanent generation at start-up; give them back so
        # that dropping the last reference (and a collection) frees the weights and the KV pool
        import gc
        gc.unfreeze()
