"""Environment access in one place: typed getters over the registered FASTINFERENCE_* / VLLM_* /
FI_* variables (names in ``config/env_names.py``, typed registry in ``config/env_registry.py``).
Reference: vllm/envs.py."""
from __future__ import annotations

import os

from .config import env_registry
from .utils.misc import truthy


def get(name: str, default=None):
    """Raw string value of a variable (``default`` when unset)."""
    return os.environ.get(name, default)


def is_registered(name: str) -> bool:
    return env_registry.is_registered(name)


def get_bool(name: str, default: bool = False) -> bool:
    raw = os.environ.get(name)
    return default if raw is None else truthy(raw)


def get_int(name: str, default: int = 0) -> int:
    raw = os.environ.get(name)
    try:
        return int(raw) if raw is not None else default
    except ValueError:
        return default


FI_USE_PDL = lambda: get_bool("FI_USE_PDL", True)                     # programmatic dependent launch
FI_BUILD_VERBOSE = lambda: get_bool("FI_BUILD_VERBOSE", False)
