"""Quantised linear weights behind one interface, the execution-policy resolver that decides which
path a layer takes, and the audit trail of those decisions.

* ``QuantizedLinearWeight.matmul(x, bias)`` is implemented by ``GGUFWeight`` (raw GGUF blocks of type
  Q8_0 / Q2_K / IQ2_XXS / Q4_0 / Q4_K / Q6_K, consumed in place by the block kernels) and by
  ``Int4LinearWeight`` (AWQ zero-point and compressed-tensors symmetric int4 in the tcgen05 runtime
  layout).  Both have a *native* path (quantised bytes stream through the kernel) and a *dense* path
  (dequantise once, keep the 16-bit copy in a byte-budgeted LRU, run the dense tensor-core GEMM).
* ``resolve_execution_policy`` turns the user's scope (``off`` / ``attention_only`` / ``all``), the
  high-fidelity prefixes and the dense-cache budget into an ``ExecutionPolicy``;
  ``should_use_native_path(prefix, policy)`` answers per layer and says why.
* ``record_audit_event`` keeps counters per path, per layer prefix and a bounded list of events
  (prefix, path, reason, shape, dtypes); ``audit_summary()`` is what the engine's stats endpoint shows.

Reference: vllm/model_executor/layers/quantization/tensor.py:53-115 (LRU cache), :290-327 (audit
events), :597-675 (policy resolver), :693-735 (stats), :946-1005 (weight classes).  There the dense
path is the default on most layers and the fused Triton path is opt-in per prefix; here the native
kernels are the default and the dense path is what a high-fidelity prefix or ``scope = off`` selects.
"""
from __future__ import annotations

import threading
from collections import OrderedDict, deque
from dataclasses import dataclass, field

import torch

from ...ops import gguf_quant as gq


# ---------------------------------------------------------------------------- dense-copy cache
class LRUWeightCache:
    """Dense 16-bit copies of quantised weights, least recently used first out, bounded by entry
    count and by bytes (0 = no byte bound)."""

    def __init__(self, max_size: int = 256, max_bytes: int = 0):
        self.max_size, self.max_bytes = int(max_size), int(max_bytes)
        self._items: OrderedDict[int, torch.Tensor] = OrderedDict()
        self.bytes_used = 0
        self.hits = self.misses = self.evictions = 0

    def get(self, key: int):
        t = self._items.get(key)
        if t is None:
            self.misses += 1
            return None
        self._items.move_to_end(key)
        self.hits += 1
        return t

    def put(self, key: int, value: torch.Tensor) -> bool:
        """False when the tensor alone exceeds the byte budget (then it is not kept)."""
        nbytes = value.numel() * value.element_size()
        if self.max_bytes and nbytes > self.max_bytes:
            return False
        old = self._items.pop(key, None)
        if old is not None:
            self.bytes_used -= old.numel() * old.element_size()
        self._items[key] = value
        self.bytes_used += nbytes
        while len(self._items) > self.max_size or (self.max_bytes and self.bytes_used > self.max_bytes):
            _, ev = self._items.popitem(last=False)
            self.bytes_used -= ev.numel() * ev.element_size()
            self.evictions += 1
        return True

    def clear(self) -> None:
        self._items.clear()
        self.bytes_used = 0

    def get_memory_stats(self) -> dict:
        return {"entries": len(self._items), "bytes": self.bytes_used, "hits": self.hits, "misses": self.misses,
                "evictions": self.evictions, "max_bytes": self.max_bytes}


_DENSE_CACHE = LRUWeightCache(max_size=256, max_bytes=8 << 30)


def dense_cache() -> LRUWeightCache:
    return _DENSE_CACHE


def clear_global_weight_cache() -> None:
    _DENSE_CACHE.clear()


# ---------------------------------------------------------------------------- policy
SCOPES = ("off", "attention_only", "all")
_ATTENTION_MARKERS = ("self_attn", "attention", ".attn.", "q_proj", "k_proj", "v_proj", "o_proj", "qkv_proj")


@dataclass(frozen=True)
class ExecutionPolicy:
    """Which layers run on their quantised bytes (``native_scope``), which must run on a dense copy
    whatever the scope (``high_fidelity_prefixes``), and whether dense copies may be cached."""
    native_scope: str = "all"
    high_fidelity_prefixes: tuple = ()
    dense_cache_enabled: bool = True
    dense_cache_max_bytes: int = 8 << 30


def is_attention_like_prefix(prefix: str) -> bool:
    p = prefix or ""
    return any(m in p for m in _ATTENTION_MARKERS)


def resolve_execution_policy(config=None, *, scope: str | None = None, high_fidelity_prefixes=(),
                             dense_cache_max_gb: float | None = None) -> ExecutionPolicy:
    """Explicit arguments win over ``config`` (an object or dict with ``quant_native_scope``,
    ``quant_high_fidelity_prefixes``, ``quant_dense_cache_max_gb``); unknown scopes are rejected."""
    def cfg(name, default):
        if config is None:
            return default
        if isinstance(config, dict):
            return config.get(name, default)
        return getattr(config, name, default)

    sc = scope if scope is not None else cfg("quant_native_scope", "all")
    if sc not in SCOPES:
        raise ValueError(f"quantised-kernel scope must be one of {SCOPES}, got {sc!r}")
    hf = tuple(high_fidelity_prefixes) or tuple(cfg("quant_high_fidelity_prefixes", ()) or ())
    gb = dense_cache_max_gb if dense_cache_max_gb is not None else cfg("quant_dense_cache_max_gb", 8.0)
    gb = float(gb)
    return ExecutionPolicy(native_scope=sc, high_fidelity_prefixes=hf, dense_cache_enabled=gb > 0,
                           dense_cache_max_bytes=int(gb * (1 << 30)))


def should_use_native_path(prefix: str, policy: ExecutionPolicy) -> tuple[bool, str]:
    """(use the quantised-byte kernel?, reason)."""
    p = prefix or ""
    for hf in policy.high_fidelity_prefixes:
        if hf and hf in p:
            return False, f"high-fidelity prefix {hf!r}"
    if policy.native_scope == "off":
        return False, "scope off"
    if policy.native_scope == "attention_only" and not is_attention_like_prefix(p):
        return False, "scope attention_only"
    return True, f"scope {policy.native_scope}"


_POLICY = ExecutionPolicy()


def set_execution_policy(policy: ExecutionPolicy) -> None:
    global _POLICY
    _POLICY = policy
    _DENSE_CACHE.max_bytes = policy.dense_cache_max_bytes if policy.dense_cache_enabled else 1


def get_execution_policy() -> ExecutionPolicy:
    return _POLICY


# ---------------------------------------------------------------------------- audit
@dataclass
class _Audit:
    enabled: bool = False
    counters: dict = field(default_factory=dict)
    by_prefix: dict = field(default_factory=dict)
    events: deque = field(default_factory=lambda: deque(maxlen=256))
    lock: threading.Lock = field(default_factory=threading.Lock)


_AUDIT = _Audit()


def enable_audit(on: bool = True, max_events: int = 256) -> None:
    """Off by default: recording costs a lock and a few dict updates per quantised matmul."""
    with _AUDIT.lock:
        _AUDIT.enabled = bool(on)
        _AUDIT.events = deque(_AUDIT.events, maxlen=max_events)


def record_audit_event(prefix: str, path: str, reason: str, *, kind: str, shape: dict | None = None,
                       dtypes: dict | None = None) -> None:
    """``path`` in {"native", "dense", "dense_cached"}; ``kind`` names the weight format."""
    if not _AUDIT.enabled:
        return
    with _AUDIT.lock:
        c = _AUDIT.counters
        c[f"{kind}.{path}"] = c.get(f"{kind}.{path}", 0) + 1
        c["calls"] = c.get("calls", 0) + 1
        row = _AUDIT.by_prefix.setdefault(prefix or "<unnamed>", {"calls": 0, "tokens": 0, "native": 0, "dense": 0})
        row["calls"] += 1
        row["tokens"] += int((shape or {}).get("m", 0))
        row["native" if path == "native" else "dense"] += 1
        _AUDIT.events.append({"prefix": prefix, "path": path, "reason": reason, "kind": kind,
                              "shape": {k: int(v) for k, v in (shape or {}).items()},
                              "dtypes": {k: str(v) for k, v in (dtypes or {}).items()}})


def reset_runtime_stats() -> None:
    with _AUDIT.lock:
        _AUDIT.counters.clear()
        _AUDIT.by_prefix.clear()
        _AUDIT.events.clear()


def runtime_stats() -> dict:
    with _AUDIT.lock:
        return dict(_AUDIT.counters)


def runtime_prefix_stats(limit: int = 20) -> dict:
    with _AUDIT.lock:
        rows = sorted(_AUDIT.by_prefix.items(), key=lambda kv: -kv[1]["calls"])[:limit]
        return {k: dict(v) for k, v in rows}


def audit_summary(limit: int = 20) -> dict:
    """Counters, the busiest prefixes, the most recent events and the dense-cache state."""
    with _AUDIT.lock:
        recent = list(_AUDIT.events)[-limit:]
    return {"enabled": _AUDIT.enabled, "policy": {"native_scope": _POLICY.native_scope,
                                                  "high_fidelity_prefixes": list(_POLICY.high_fidelity_prefixes),
                                                  "dense_cache_enabled": _POLICY.dense_cache_enabled},
            "counters": runtime_stats(), "prefixes": runtime_prefix_stats(limit), "recent_events": recent,
            "dense_cache": _DENSE_CACHE.get_memory_stats()}


# ---------------------------------------------------------------------------- weights
class QuantizedLinearWeight:
    """A quantised ``[N, K]`` weight.  ``matmul(x, bias)`` returns ``x @ W.T (+ bias)``."""
    kind = "quantized"

    def __init__(self, prefix: str = ""):
        self.prefix = prefix

    @property
    def shape(self) -> tuple[int, int]:
        raise NotImplementedError

    def dense(self, dtype: torch.dtype) -> torch.Tensor:
        raise NotImplementedError

    def _native(self, x, residual, out_dtype):
        raise NotImplementedError

    def _cached_dense(self, dtype: torch.dtype, policy: ExecutionPolicy) -> tuple[torch.Tensor, bool]:
        key = (id(self) << 4) ^ hash(dtype)
        if policy.dense_cache_enabled:
            w = _DENSE_CACHE.get(key)
            if w is not None:
                return w, True
        w = self.dense(dtype)
        if policy.dense_cache_enabled:
            _DENSE_CACHE.put(key, w)
        return w, False

    def matmul(self, x: torch.Tensor, bias: torch.Tensor | None = None, *, residual: torch.Tensor | None = None,
               out_dtype: torch.dtype | None = None, policy: ExecutionPolicy | None = None) -> torch.Tensor:
        from ... import ops
        policy = policy or _POLICY
        native, reason = should_use_native_path(self.prefix, policy)
        N, K = self.shape
        shape = {"m": x.shape[0], "n": N, "k": K}
        if native:
            y = self._native(x, residual, out_dtype)
            if bias is not None:
                y = y + bias.to(y.dtype)
            record_audit_event(self.prefix, "native", reason, kind=self.kind, shape=shape,
                               dtypes={"x": x.dtype, "out": y.dtype})
            return y
        w, hit = self._cached_dense(x.dtype if x.dtype != torch.float32 or not x.is_cuda else torch.bfloat16, policy)
        xin = x if x.dtype == w.dtype else x.to(w.dtype)
        y = ops.linear(xin, w, bias, residual, out_dtype=out_dtype)
        record_audit_event(self.prefix, "dense_cached" if hit else "dense", reason, kind=self.kind, shape=shape,
                           dtypes={"x": x.dtype, "w": w.dtype, "out": y.dtype})
        return y


class GGUFWeight(QuantizedLinearWeight):
    """Raw GGUF blocks ``uint8 [N, row_bytes]`` of one block type (Q4_0, Q4_K, Q6_K, Q8_0, Q2_K,
    IQ2_XXS).  Native path: the block-streaming GEMV for up to 8 rows of ``x``, beyond that one
    dequantisation into scratch plus the tensor-core GEMM (``ops.gguf_quant.gguf_linear``)."""
    kind = "gguf"

    def __init__(self, raw: torch.Tensor, ggml_type: int | str, in_features: int, prefix: str = ""):
        super().__init__(prefix)
        ty = gq.GGML_TYPES[ggml_type] if isinstance(ggml_type, str) else int(ggml_type)
        if ty not in gq.BLOCK:
            raise ValueError(f"GGUF block type {ggml_type!r} is not a supported weight format "
                             f"(supported: {sorted(gq.TYPE_NAMES[t] for t in gq.BLOCK)})")
        if raw.dtype != torch.uint8 or raw.dim() != 2 or raw.shape[1] != gq.row_bytes(ty, in_features):
            raise ValueError(f"raw blocks must be uint8 [N, {gq.row_bytes(ty, in_features)}] for K={in_features}, "
                             f"got {tuple(raw.shape)} {raw.dtype}")
        self.raw, self.ggml_type, self.in_features = raw.contiguous(), ty, int(in_features)

    @property
    def shape(self) -> tuple[int, int]:
        return self.raw.shape[0], self.in_features

    def to(self, device) -> "GGUFWeight":
        self.raw = self.raw.to(device)
        return self

    def dense(self, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        if self.raw.is_cuda and dtype in (torch.bfloat16, torch.float16):
            return gq.dequantize_cuda(self.raw, self.ggml_type, self.in_features, dtype)
        return gq.dequantize(self.raw, self.ggml_type, self.in_features).to(dtype)

    def _native(self, x, residual, out_dtype):
        return gq.gguf_linear(x, self.raw, self.ggml_type, self.in_features, residual=residual, out_dtype=out_dtype)


class Int4LinearWeight(QuantizedLinearWeight):
    """AWQ (zero-point, group 128) or compressed-tensors (symmetric, group 32) int4 weight wrapped
    around :class:`litevllm_b200.ops.awq.Int4Weight`."""
    kind = "int4"

    def __init__(self, int4, prefix: str = ""):
        super().__init__(prefix)
        self.int4 = int4

    @property
    def shape(self) -> tuple[int, int]:
        return self.int4.N, self.int4.K

    def dense(self, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        return self.int4.dense().to(dtype)

    def _native(self, x, residual, out_dtype):
        from ...ops import awq
        return awq.int4_linear(x, self.int4, residual=residual, out_dtype=out_dtype)
