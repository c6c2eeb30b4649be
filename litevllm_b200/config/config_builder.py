"""``build_vllm_config(model, **kwargs) -> VllmConfig``.

Accepted ``model`` forms: a checkpoint directory with ``config.json`` (safetensors, AWQ or
compressed-tensors), a ``.gguf`` file, or ``synthetic:<preset>`` (random-init weights of a named
architecture).  Keyword contract follows vllm/serving/config_builder.py:139-227 of the reference:
``max_model_len, gpu_memory_utilization, max_num_seqs|concurrent_reqs, max_num_batched_tokens, dtype,
tokenizer, cache_block_size, policy_mode, trust_remote_code, revision, fastinference_config,
fastinference_config_path`` plus ``tensor_parallel_size, expert_parallel_size, comm_backend, seed,
hf_overrides, load_format, device``.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any

from ..models.arch import arch_from_hf_config
from ..models.presets import get_preset
from .fastinference_config import resolve_fastinference_config
from .model_config import (CacheConfig, LoadConfig, ModelConfig, SchedulerConfig, VllmConfig,
                           resolve_dtype)
from .parallel_config import ParallelConfig
from .runtime_config import RuntimeConfig

_KNOWN_KW = {
    "fastinference_config", "fastinference_config_path", "trust_remote_code", "revision",
    "max_model_len", "gpu_memory_utilization", "max_num_seqs", "concurrent_reqs",
    "max_num_batched_tokens", "tokenizer", "dtype", "cache_block_size", "policy_mode",
    "tensor_parallel_size", "expert_parallel_size", "data_parallel_size", "comm_backend", "seed", "hf_overrides",
    "load_format", "device", "quantization", "enforce_eager",
}


def _deep_update(dst: dict, src: dict) -> dict:
    for k, v in src.items():
        if isinstance(v, dict) and isinstance(dst.get(k), dict):
            _deep_update(dst[k], v)
        else:
            dst[k] = v
    return dst


def load_hf_config_dict(model: str) -> tuple[dict, bool, bool]:
    """-> (config dict, is_gguf, synthetic)."""
    if model.startswith("synthetic:"):
        return get_preset(model.split(":", 1)[1]), False, True
    p = Path(model)
    if p.is_file() and p.suffix == ".gguf":
        from ..loaders.gguf import hf_config_from_gguf
        return hf_config_from_gguf(p), True, False
    if p.is_dir():
        cfg_file = p / "config.json"
        if cfg_file.is_file():
            cfg = json.loads(cfg_file.read_text())
            qfile = p / "hf_quant_config.json"
            if qfile.is_file() and "quantization_config" not in cfg:
                cfg["quantization_config"] = json.loads(qfile.read_text()).get("quantization", {}) or \
                    {"quant_method": "awq"}
            ggufs = sorted(p.glob("*.gguf"))
            return cfg, bool(ggufs) and not list(p.glob("*.safetensors")), False
        ggufs = sorted(p.glob("*.gguf"))
        if ggufs:
            from ..loaders.gguf import hf_config_from_gguf
            return hf_config_from_gguf(ggufs[0]), True, False
    raise FileNotFoundError(
        f"cannot resolve model {model!r}: expected a directory with config.json, a .gguf file or "
        f"synthetic:<preset> (remote hub ids are not downloaded by this engine)")


def make_quant_config(arch, hf_cfg: dict):
    from ..layers.quantization import get_quantization_config
    return get_quantization_config(arch.quant, hf_cfg)


def build_vllm_config(model: str, **kwargs: Any) -> VllmConfig:
    unknown = sorted(set(kwargs) - _KNOWN_KW)
    if unknown:
        raise TypeError(f"build_vllm_config got unexpected keyword(s): {', '.join(unknown)}")
    fi = resolve_fastinference_config(config=kwargs.get("fastinference_config"),
                                      path=kwargs.get("fastinference_config_path"))
    trust = bool(kwargs.get("trust_remote_code", fi.model.trust_remote_code))
    revision = kwargs.get("revision", fi.model.revision)
    if trust and not revision:
        raise ValueError("trust_remote_code requires a pinned revision")

    hf_cfg, is_gguf, synthetic = load_hf_config_dict(str(model))
    if kwargs.get("hf_overrides"):
        _deep_update(hf_cfg, dict(kwargs["hf_overrides"]))
    if kwargs.get("load_format") == "dummy":
        synthetic = True
    arch = arch_from_hf_config(hf_cfg)

    dtype = resolve_dtype(kwargs.get("dtype") or hf_cfg.get("torch_dtype") or hf_cfg.get("dtype") or "bfloat16")
    max_len = int(kwargs.get("max_model_len") or min(arch.max_position, 4096))
    seqs = int(kwargs.get("max_num_seqs") or kwargs.get("concurrent_reqs") or 8)
    batched = int(kwargs.get("max_num_batched_tokens") or max(8192, seqs * min(max_len, 1024)))
    parallel = ParallelConfig.from_env(
        tp=int(kwargs.get("tensor_parallel_size") or fi.parallel.tensor_parallel_size),
        ep=int(kwargs.get("expert_parallel_size") or fi.parallel.expert_parallel_size),
        dp=int(kwargs.get("data_parallel_size") or 1),
        comm_backend=str(kwargs.get("comm_backend") or fi.parallel.comm_backend))

    cfg = VllmConfig(
        model_config=ModelConfig(model=str(model), tokenizer=str(kwargs.get("tokenizer") or model),
                                 dtype=dtype, max_model_len=max_len, arch=arch, hf_config=hf_cfg,
                                 trust_remote_code=trust, revision=revision, is_gguf=is_gguf,
                                 synthetic=synthetic, seed=int(kwargs.get("seed") or 0)),
        cache_config=CacheConfig(block_size=int(kwargs.get("cache_block_size") or 16),
                                 gpu_memory_utilization=float(kwargs.get("gpu_memory_utilization") or 0.90)),
        scheduler_config=SchedulerConfig(max_num_seqs=seqs, max_num_batched_tokens=batched,
                                         max_model_len=max_len),
        load_config=LoadConfig(load_format=str(kwargs.get("load_format") or "auto"),
                               device=str(kwargs.get("device") or "auto")),
        parallel_config=parallel, fastinference_config=fi, device=str(kwargs.get("device") or "auto"))
    cfg.quant_config = make_quant_config(arch, hf_cfg)
    cfg.runtime_config = RuntimeConfig.from_vllm_config(cfg, policy_mode=str(kwargs.get("policy_mode") or "auto"))
    return cfg
