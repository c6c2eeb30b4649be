"""Platform description.  One platform exists: NVIDIA Blackwell (sm_100a) through CUDA; CPU tensors
run the PyTorch reference ops.  Reference: vllm/platforms/__init__.py (a stub that reports "cuda")."""
from __future__ import annotations

import torch


class CudaPlatform:
    device_name = "cuda"
    device_type = "cuda"
    arch = "sm_100a"

    @staticmethod
    def is_available() -> bool:
        return torch.cuda.is_available()

    @staticmethod
    def device_count() -> int:
        return torch.cuda.device_count() if torch.cuda.is_available() else 0

    @staticmethod
    def total_memory(index: int = 0) -> int:
        return torch.cuda.get_device_properties(index).total_memory

    @staticmethod
    def is_blackwell(index: int = 0) -> bool:
        return torch.cuda.is_available() and torch.cuda.get_device_capability(index)[0] == 10


current_platform = CudaPlatform()
