"""Logging setup: one stderr handler, level from ``FASTINFERENCE_LOG_LEVEL`` / ``VLLM_LOGGING_LEVEL``
(reference: vllm/logger.py:5-17)."""
from __future__ import annotations

import logging
import os
import sys

_FORMAT = "%(levelname)s %(asctime)s %(name)s] %(message)s"
_configured = False


def _configure_root() -> None:
    global _configured
    if _configured:
        return
    root = logging.getLogger("litevllm_b200")
    level = os.environ.get("FASTINFERENCE_LOG_LEVEL") or os.environ.get("VLLM_LOGGING_LEVEL") or "INFO"
    root.setLevel(getattr(logging, level.upper(), logging.INFO))
    if not root.handlers:
        h = logging.StreamHandler(sys.stderr)
        h.setFormatter(logging.Formatter(_FORMAT, datefmt="%m-%d %H:%M:%S"))
        root.addHandler(h)
    root.propagate = False
    _configured = True


def init_logger(name: str) -> logging.Logger:
    _configure_root()
    if not name.startswith("litevllm_b200"):
        name = "litevllm_b200." + name
    return logging.getLogger(name)


def set_log_level(level: str) -> None:
    _configure_root()
    logging.getLogger("litevllm_b200").setLevel(getattr(logging, str(level).upper(), logging.INFO))
