"""Collects what the runtime factory needs from a half-built engine (model, plans, policies, adapter
supplied components) into one context object.
Reference: vllm/engine/initialization/runtime_component_factory.py:19-99."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from ..custom_runtime_components import CustomRuntimeComponents
from ..kv_cache import KVLayerSpec


@dataclass
class RuntimeAssemblyContext:
    model: Any
    arch: Any
    device: torch.device
    runtime_config: Any
    inference_config: Any
    model_policy: Any
    capabilities: Any
    plan: Any
    kv_plan: Any
    kv_specs: list
    observer: Any
    custom: CustomRuntimeComponents | None
    on_release: Any = None


class LiteRuntimeAssembler:
    @staticmethod
    def assemble(engine, planner, device_total_bytes: int | None) -> RuntimeAssemblyContext:
        plan = planner.build_execution_plan(device_total_bytes)
        engine.plan = plan                       # adapters may look at the plan while building executors
        custom = engine.adapter.build_executors(engine)
        if custom is not None and not isinstance(custom, CustomRuntimeComponents):
            custom = CustomRuntimeComponents(getattr(custom, "prefill_executor", None),
                                             getattr(custom, "decode_executor", None),
                                             getattr(custom, "kv_block_manager", None))
        specs = [s if isinstance(s, KVLayerSpec) else KVLayerSpec(*s) for s in engine.model.kv_cache_specs()]
        kv_plan = planner.build_kv_cache_plan(plan, specs, engine.model_config.dtype,
                                              engine.model_policy.force_kv_cache_dtype)
        return RuntimeAssemblyContext(
            model=engine.model, arch=engine.arch, device=engine.device, runtime_config=engine.rc,
            inference_config=engine.inf_config, model_policy=engine.model_policy, capabilities=engine.capabilities,
            plan=plan, kv_plan=kv_plan, kv_specs=specs, observer=engine.observer, custom=custom,
            on_release=engine._on_release)
