"""Config holders assembled by ``build_vllm_config`` (reference: vllm/config/{vllm,model,cache,
scheduler,load}.py).  They are plain records; policy lives in :class:`RuntimeConfig`."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

from ..models.arch import ModelArch
from .fastinference_config import FastInferenceConfig
from .parallel_config import ParallelConfig

_DTYPES = {"float16": torch.float16, "half": torch.float16, "fp16": torch.float16,
           "bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "float": torch.float32, "fp32": torch.float32}


def resolve_dtype(name: Any) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    key = str(name).replace("torch.", "").lower()
    if key not in _DTYPES:
        raise ValueError(f"unsupported dtype {name!r}")
    return _DTYPES[key]


@dataclass
class ModelConfig:
    model: str
    tokenizer: str
    dtype: torch.dtype
    max_model_len: int
    arch: ModelArch
    hf_config: dict[str, Any] = field(default_factory=dict)
    trust_remote_code: bool = False
    revision: str | None = None
    is_gguf: bool = False
    synthetic: bool = False          # random-init weights of this architecture (benchmarks/tests)
    seed: int = 0

    def get_num_layers(self, parallel_config: ParallelConfig | None = None) -> int:
        return self.arch.num_layers

    def get_num_kv_heads(self, parallel_config: ParallelConfig | None = None) -> int:
        tp = parallel_config.tensor_parallel_size if parallel_config else 1
        return max(1, self.arch.num_kv_heads // tp)

    def get_head_size(self) -> int:
        return self.arch.head_dim

    def get_vocab_size(self) -> int:
        return self.arch.vocab_size


@dataclass
class CacheConfig:
    block_size: int = 16
    gpu_memory_utilization: float = 0.90
    cache_dtype: str = "auto"


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 8
    max_num_batched_tokens: int = 8192
    max_model_len: int = 4096


@dataclass
class LoadConfig:
    load_format: str = "auto"
    device: str = "auto"


@dataclass
class ObservabilityConfig:
    otlp_traces_endpoint: str | None = None
    collect_detailed_traces: bool = False


@dataclass
class MultiModalConfig:
    limit_per_prompt: dict[str, int] = field(default_factory=lambda: {"image": 4})


@dataclass
class VllmConfig:
    model_config: ModelConfig
    cache_config: CacheConfig
    scheduler_config: SchedulerConfig
    load_config: LoadConfig
    parallel_config: ParallelConfig
    fastinference_config: FastInferenceConfig
    quant_config: Any = None
    runtime_config: Any = None
    observability_config: ObservabilityConfig = field(default_factory=ObservabilityConfig)
    multimodal_config: MultiModalConfig = field(default_factory=MultiModalConfig)
    device: str = "auto"
