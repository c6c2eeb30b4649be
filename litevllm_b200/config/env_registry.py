"""Registry of setting names with a scope each.

Only ``FASTINFERENCE_CONFIG`` is a public process-environment variable; everything else reaches the
engine through the TOML file's ``[tuning_keyvals]`` table.  Deprecated names may additionally be
read from the environment when ``FASTINFERENCE_ALLOW_LEGACY_ENV`` is truthy.
Behavioural contract: vllm/engine/env_registry.py:9-691 of the reference.
"""
from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass
from enum import Enum

from . import env_names

PREFIX = "FASTINFERENCE_"


class EnvScope(str, Enum):
    PUBLIC = "public"
    DEPRECATED = "deprecated"
    TOOL_ONLY = "tool_only"
    REMOVED = "removed"
    NEW = "new"  # multi-GPU / B200 additions, TOML only


@dataclass(frozen=True)
class EnvSpec:
    name: str
    scope: EnvScope
    replacement: str | None = None


def _build() -> dict[str, EnvSpec]:
    reg: dict[str, EnvSpec] = {}
    groups = ((env_names.PUBLIC, EnvScope.PUBLIC), (env_names.REMOVED, EnvScope.REMOVED),
              (env_names.DEPRECATED, EnvScope.DEPRECATED), (env_names.TOOL_ONLY, EnvScope.TOOL_ONLY),
              (env_names.NEW, EnvScope.NEW))
    for blob, scope in groups:
        for short in blob.split():
            name = PREFIX + short
            repl = "TOML profile / [tuning_keyvals]" if scope is EnvScope.DEPRECATED else None
            reg[name] = EnvSpec(name, scope, repl)
    return reg


ENV_REGISTRY: dict[str, EnvSpec] = _build()
PUBLIC_ENV_NAMES = frozenset(n for n, s in ENV_REGISTRY.items() if s.scope is EnvScope.PUBLIC)

_TRUE = {"1", "true", "yes", "on"}


def truthy(value: object) -> bool:
    return str(value).strip().lower() in _TRUE


def is_registered(name: str) -> bool:
    return name in ENV_REGISTRY


def is_usable_tuning_key(name: str) -> bool:
    spec = ENV_REGISTRY.get(name)
    return spec is not None and spec.scope is not EnvScope.REMOVED


def legacy_env_enabled(environ: Mapping[str, str]) -> bool:
    return truthy(environ.get(PREFIX + "ALLOW_LEGACY_ENV", ""))


def collect_legacy_tuning_env(environ: Mapping[str, str], *, require_flag: bool = True) -> dict[str, str]:
    """Deprecated-scope names found in ``environ`` (empty unless the legacy switch is on)."""
    if require_flag and not legacy_env_enabled(environ):
        return {}
    return {k: v for k, v in environ.items()
            if k in ENV_REGISTRY and ENV_REGISTRY[k].scope is EnvScope.DEPRECATED}


def get_public_env(environ: Mapping[str, str], name: str, default: str = "") -> str:
    spec = ENV_REGISTRY.get(name)
    if spec is None or spec.scope is not EnvScope.PUBLIC:
        raise ValueError(f"{name} is not a public environment variable of this engine")
    return environ.get(name, default)


def kernel_switches() -> dict[str, str]:
    """The ``FI_*`` process-environment switches of the kernel layer with what each selects."""
    return dict(env_names.KERNEL_SWITCHES)
