"""TOML user configuration (``FASTINFERENCE_CONFIG=<file>``).

Schema (unknown keys are errors; contract: vllm/engine/fastinference_config.py:13-153 of the
reference, extended with a ``[parallel]`` table for multi-GPU serving)::

    profile  = "auto" | "balanced" | "latency" | "throughput" | "accuracy" | "benchmark"
    kv_type  = "auto" | "fp16" | "fp8" | "fp8_block" | "turbo_int4"
    debug    = false
    log_level = "info"
    [benchmark]      profile = "default"
    [legacy_env]     enabled = false
    [model]          trust_remote_code = false ; revision = "<sha>"
    [parallel]       tensor_parallel_size = 1 ; expert_parallel_size = 1 ; comm_backend = "fused"|"nccl"
    [tuning_keyvals] FASTINFERENCE_<NAME> = "<value>"   (registered names only)
"""
from __future__ import annotations

import os
import tomllib
from collections.abc import Mapping
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

from .env_registry import is_usable_tuning_key

PROFILES = ("auto", "balanced", "latency", "throughput", "accuracy", "benchmark")
KV_TYPES = ("auto", "fp16", "fp8", "fp8_block", "turbo_int4")
COMM_BACKENDS = ("fused", "nccl")


@dataclass(frozen=True)
class BenchmarkConfig:
    profile: str = "default"


@dataclass(frozen=True)
class LegacyEnvConfig:
    enabled: bool = False


@dataclass(frozen=True)
class ModelLoadConfig:
    trust_remote_code: bool = False
    revision: str | None = None


@dataclass(frozen=True)
class ParallelTomlConfig:
    tensor_parallel_size: int = 1
    expert_parallel_size: int = 1
    comm_backend: str = "fused"


@dataclass(frozen=True)
class FastInferenceConfig:
    profile: str = "auto"
    kv_type: str = "auto"
    debug: bool = False
    log_level: str = "info"
    benchmark: BenchmarkConfig = field(default_factory=BenchmarkConfig)
    legacy_env: LegacyEnvConfig = field(default_factory=LegacyEnvConfig)
    model: ModelLoadConfig = field(default_factory=ModelLoadConfig)
    parallel: ParallelTomlConfig = field(default_factory=ParallelTomlConfig)
    tuning_keyvals: dict[str, str] = field(default_factory=dict)


def _table(data: Mapping[str, Any], key: str, allowed: tuple[str, ...]) -> Mapping[str, Any]:
    value = data.get(key)
    if value is None:
        return {}
    if not isinstance(value, Mapping):
        raise ValueError(f"[{key}] must be a table")
    extra = sorted(set(value) - set(allowed))
    if extra and key != "tuning_keyvals":
        raise ValueError(f"Unknown keys in [{key}]: {', '.join(extra)}")
    return value


def _choice(value: Any, choices: tuple[str, ...], what: str, default: str) -> str:
    text = str(value if value is not None else default).strip().lower() or default
    if text not in choices:
        raise ValueError(f"{what} must be one of {sorted(choices)} (got {text!r})")
    return text


def _positive_int(value: Any, what: str) -> int:
    try:
        n = int(value)
    except (TypeError, ValueError):
        raise ValueError(f"{what} must be an integer") from None
    if n < 1:
        raise ValueError(f"{what} must be >= 1")
    return n


_TOP_LEVEL = ("profile", "kv_type", "debug", "log_level", "benchmark", "legacy_env", "model",
              "parallel", "tuning_keyvals")


def config_from_mapping(data: Mapping[str, Any]) -> FastInferenceConfig:
    extra = sorted(set(data) - set(_TOP_LEVEL))
    if extra:
        raise ValueError("Unknown FastInference config fields: " + ", ".join(extra))
    bench = _table(data, "benchmark", ("profile",))
    legacy = _table(data, "legacy_env", ("enabled",))
    model = _table(data, "model", ("trust_remote_code", "revision"))
    par = _table(data, "parallel", ("tensor_parallel_size", "expert_parallel_size", "comm_backend"))
    tuning = _table(data, "tuning_keyvals", ())
    keyvals = {str(k): str(v) for k, v in tuning.items()}
    bad = sorted(k for k in keyvals if not is_usable_tuning_key(k))
    if bad:
        raise ValueError("Unknown tuning_keyvals: " + ", ".join(bad))
    trust = bool(model.get("trust_remote_code", False))
    revision = str(model.get("revision", "") or "").strip() or None
    if trust and revision is None:
        raise ValueError("model.revision is required when trust_remote_code is enabled")
    return FastInferenceConfig(
        profile=_choice(data.get("profile"), PROFILES, "profile", "auto"),
        kv_type=_choice(data.get("kv_type"), KV_TYPES, "kv_type", "auto"),
        debug=bool(data.get("debug", False)),
        log_level=str(data.get("log_level", "info")).strip().lower() or "info",
        benchmark=BenchmarkConfig(str(bench.get("profile", "default")).strip().lower() or "default"),
        legacy_env=LegacyEnvConfig(bool(legacy.get("enabled", False))),
        model=ModelLoadConfig(trust, revision),
        parallel=ParallelTomlConfig(
            _positive_int(par.get("tensor_parallel_size", 1), "parallel.tensor_parallel_size"),
            _positive_int(par.get("expert_parallel_size", 1), "parallel.expert_parallel_size"),
            _choice(par.get("comm_backend"), COMM_BACKENDS, "parallel.comm_backend", "fused")),
        tuning_keyvals=keyvals,
    )


def load_fastinference_config(path: str | Path | None) -> FastInferenceConfig:
    if path is None:
        return FastInferenceConfig()
    p = Path(path).expanduser()
    if not p.is_file():
        raise FileNotFoundError(f"FastInference config file not found: {p}")
    with p.open("rb") as fh:
        return config_from_mapping(tomllib.load(fh))


def resolve_fastinference_config(*, config: FastInferenceConfig | Mapping[str, Any] | None = None,
                                 path: str | Path | None = None,
                                 environ: Mapping[str, str] | None = None) -> FastInferenceConfig:
    """Precedence: explicit object/mapping > explicit path > ``FASTINFERENCE_CONFIG`` > defaults."""
    if isinstance(config, FastInferenceConfig):
        return config
    if isinstance(config, Mapping):
        return config_from_mapping(config)
    if path is None:
        env = os.environ if environ is None else environ
        path = str(env.get("FASTINFERENCE_CONFIG", "")).strip() or None
    return load_fastinference_config(path)
