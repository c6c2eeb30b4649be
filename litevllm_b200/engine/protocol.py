"""Abstract client interface implemented by ``AsyncLLM`` (reference: vllm/engine/protocol.py:9-34)."""
from __future__ import annotations

from abc import ABC, abstractmethod


class EngineClient(ABC):
    @abstractmethod
    def generate(self, prompt, sampling_params, request_id, lora_request=None, multi_modal_data=None): ...

    @abstractmethod
    async def abort(self, request_id) -> None: ...

    @abstractmethod
    def is_healthy(self) -> bool: ...

    @abstractmethod
    def shutdown(self) -> None: ...
