"""Small helpers (reference: vllm/utils/*)."""
from __future__ import annotations

from collections import OrderedDict
from typing import Any, Generic, Hashable, TypeVar

import torch

K = TypeVar("K", bound=Hashable)
V = TypeVar("V")


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def round_up(a: int, b: int) -> int:
    return cdiv(a, b) * b


def dtype_nbytes(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def truthy(value: Any) -> bool:
    return str(value).strip().lower() in {"1", "true", "yes", "on"}


class LRUCache(Generic[K, V]):
    def __init__(self, capacity: int):
        self.capacity = max(0, int(capacity))
        self._d: OrderedDict[K, V] = OrderedDict()

    def get(self, key: K, default: V | None = None) -> V | None:
        if key in self._d:
            self._d.move_to_end(key)
            return self._d[key]
        return default

    def put(self, key: K, value: V) -> None:
        if self.capacity == 0:
            return
        self._d[key] = value
        self._d.move_to_end(key)
        while len(self._d) > self.capacity:
            self._d.popitem(last=False)

    def pop(self, key: K, default=None):
        return self._d.pop(key, default)

    def clear(self) -> None:
        self._d.clear()

    def __len__(self) -> int:
        return len(self._d)

    def __contains__(self, key: K) -> bool:
        return key in self._d

    def items(self):
        return self._d.items()
