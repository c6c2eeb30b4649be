"""Runtime registry of LoRA adapters: name -> loaded adapter, active reference counts, and the
per-batch mapping handed to the linear layers.  Reference: vllm/engine/lora_runtime.py:21-128."""
from __future__ import annotations

from dataclasses import dataclass

from .errors import InvalidRequestError


@dataclass(frozen=True)
class LoRARequest:
    lora_name: str
    lora_int_id: int = 0
    lora_path: str = ""


class LoRARuntimeRegistry:
    def __init__(self, model, device):
        from ..lora.manager import LoRAManager
        self.manager = LoRAManager(model, device)
        self.requests: dict[str, LoRARequest] = {}
        self.active: dict[str, int] = {}
        self._next_id = 1

    def register(self, lora_name: str, lora_path: str, lora_int_id: int | None = None) -> LoRARequest:
        if lora_name in self.requests:
            return self.requests[lora_name]
        if lora_int_id is None:
            lora_int_id = self._next_id
        self._next_id = max(self._next_id, lora_int_id) + 1
        self.manager.load_adapter(lora_name, lora_path)
        req = LoRARequest(lora_name, lora_int_id, lora_path)
        self.requests[lora_name] = req
        return req

    def unregister(self, lora_name: str) -> bool:
        if self.active.get(lora_name, 0) > 0:
            raise InvalidRequestError(f"LoRA adapter {lora_name!r} is in use by running requests")
        if self.requests.pop(lora_name, None) is None:
            return False
        self.manager.remove_adapter(lora_name)
        return True

    def resolve(self, lora_request) -> LoRARequest:
        name = lora_request if isinstance(lora_request, str) else getattr(lora_request, "lora_name", None)
        if name not in self.requests:
            raise InvalidRequestError(f"unknown LoRA adapter {name!r}")
        return self.requests[name]

    def acquire(self, lora_request) -> None:
        req = self.resolve(lora_request)
        self.active[req.lora_name] = self.active.get(req.lora_name, 0) + 1

    def release(self, lora_request) -> None:
        name = lora_request if isinstance(lora_request, str) else getattr(lora_request, "lora_name", None)
        if name in self.active:
            self.active[name] -= 1
            if self.active[name] <= 0:
                del self.active[name]

    def _name_of(self, st) -> str | None:
        lr = st.lora_request
        if lr is None:
            return None
        return lr if isinstance(lr, str) else lr.lora_name

    def mapping_for_prefill(self, items, states):
        names = [self._name_of(states[it.request_id]) for it in items]
        if not any(names):
            return None
        from ..lora.mapping import LoRAMapping
        return LoRAMapping.from_segments(names, [it.chunk_len for it in items])

    def mapping_for_decode(self, reqs):
        names = [self._name_of(st) for st in reqs]
        if not any(names):
            return None
        from ..lora.mapping import LoRAMapping
        return LoRAMapping.from_segments(names, [1] * len(reqs))

    def stats(self) -> dict:
        return {"registered": sorted(self.requests), "active": dict(self.active)}
