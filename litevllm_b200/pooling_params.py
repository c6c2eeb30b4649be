"""Placeholder kept for import parity (vllm/pooling_params.py in the reference is an unused stub:
the engine serves generation only)."""
from dataclasses import dataclass


@dataclass
class PoolingParams:
    additional_data: dict | None = None
