"""Wires the runtime of one rank from an assembly context: KV pool and block manager, batch builder,
multimodal processor, executors, step scheduler, prefix cache, sampling, output pipeline, backend and
controller.  Components supplied by the model adapter replace the stock ones.
Reference: vllm/engine/runtime_factory.py:35-186."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .backend import LiteGpuBackend
from .block_allocator import BlockAllocator
from .executors import DecodeExecutor, PrefillExecutor
from .initialization.runtime_component_factory import RuntimeAssemblyContext
from .input_batch import InputBatchBuilder
from .kv_block_manager import KVBlockManager
from .kv_cache import FlatKVCache
from .output_pipeline import GenerationPolicies, OutputPipeline
from .prefix_cache import PrefixCache
from .request_scheduler import RequestScheduler
from .runtime_controller import RuntimeController
from .sampling_driver import SamplingDriver
from .step_scheduler import StepScheduler


@dataclass
class RuntimeComponents:
    kv_cache: Any
    allocator: Any
    kv_manager: Any
    scheduler: Any
    builder: Any
    lora_registry: Any
    multimodal: Any
    prefill_executor: Any
    decode_executor: Any
    step_scheduler: Any
    prefix_cache: Any
    sampling_driver: Any
    output_pipeline: Any
    backend: Any
    controller: Any


class LiteRuntimeFactory:
    @staticmethod
    def build(ctx: RuntimeAssemblyContext) -> RuntimeComponents:
        plan, rc, custom = ctx.plan, ctx.runtime_config, ctx.custom
        kv_cache = FlatKVCache(ctx.kv_specs, plan.num_total_blocks, plan.block_size, ctx.kv_plan.dtype, ctx.device,
                               fmt=getattr(ctx.kv_plan, "fmt", 0))
        allocator = BlockAllocator(plan.num_total_blocks)
        kv_manager = KVBlockManager(allocator, plan.block_size, plan.max_active_requests, plan.num_blocks_per_seq,
                                    ctx.device, kv_cache)
        if custom is not None and custom.kv_block_manager is not None:
            kv_manager = custom.kv_block_manager
        scheduler = RequestScheduler(plan.max_active_requests, rc.queue_timeout_s)
        builder = InputBatchBuilder(kv_manager, plan.max_active_requests, plan.step_token_budget, ctx.device,
                                    ctx.inference_config)
        lora_registry = None
        if ctx.capabilities.supports_lora:
            from .lora_runtime import LoRARuntimeRegistry
            lora_registry = LoRARuntimeRegistry(ctx.model, ctx.device)
        multimodal = None
        if ctx.capabilities.supports_multimodal:
            from .multimodal_processor import MultimodalProcessor
            multimodal = MultimodalProcessor(ctx.arch, ctx.model)
        prefill_executor = (custom.prefill_executor if custom and custom.prefill_executor else
                            PrefillExecutor(ctx.model, kv_cache, builder, multimodal))
        decode_executor = (custom.decode_executor if custom and custom.decode_executor else
                           DecodeExecutor(ctx.model, kv_cache, builder,
                                          rc.backend_policy.cuda_graph_decode and ctx.capabilities.supports_cuda_graph))
        step_scheduler = StepScheduler(
            plan.step_token_budget, plan.prefill_chunk_size, plan.prefill_microbatch, rc.scheduler_policy,
            rc.enable_decode_priority, rc.prefill_catchup_ratio, rc.prefill_reserved_tokens,
            rc.prefill_reserve_backlog, rc.min_prefill_chunk_size, rc.max_prefill_chunk_size,
            ctx.model_policy.verified_decode_batch_sizes, plan.max_active_requests)
        prefix_cache = PrefixCache(rc.backend_policy.max_prefix_cache_entries, rc.backend_policy.max_prefix_cache_bytes)
        sampling_driver = SamplingDriver(ctx.arch.vocab_size)
        output_pipeline = OutputPipeline(None, plan.max_model_len, GenerationPolicies())
        backend = LiteGpuBackend(scheduler, kv_manager, prefill_executor, decode_executor, sampling_driver,
                                 output_pipeline, ctx.observer, rc.backend_policy, prefix_cache, lora_registry,
                                 on_release=ctx.on_release)
        controller = RuntimeController(scheduler, step_scheduler, backend, ctx.observer)
        return RuntimeComponents(kv_cache, allocator, kv_manager, scheduler, builder, lora_registry, multimodal,
                                 prefill_executor, decode_executor, step_scheduler, prefix_cache, sampling_driver,
                                 output_pipeline, backend, controller)
