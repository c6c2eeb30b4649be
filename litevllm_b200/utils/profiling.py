"""Profiling spans: NVTX ranges plus CUDA-event timers per named scope.

``with span("decode_step"): ...`` costs nothing when profiling is off.  When on, a scope pushes an
NVTX range (visible in Nsight Systems) and records a CUDA event pair on the current stream; the
event pairs are resolved lazily in ``summary()`` (one synchronise there, none in the hot path), so
spans can stay enabled while timing a run.  ``summary()`` returns ``{scope: {time_s, count}}``.
Switches: ``RuntimeConfig.profile_step_events`` / ``profile_nvtx`` (TOML ``[runtime]`` keys or the
``FASTINFERENCE_PROFILE_STEP_EVENTS`` / ``FASTINFERENCE_PROFILE_NVTX`` tuning keys) and
``bench.py --profile-json``.
Reference: vllm/model_executor/models/gemma4/profiling.py:30-97 (synchronising wall-clock spans with
optional roctx ranges) and vllm/model_executor/models/deepseek_v4_flash/profiler.py:35-151.
"""
from __future__ import annotations

import atexit
import contextlib
import json
import time

import torch


class SpanProfiler:
    def __init__(self):
        self.enabled = False
        self.nvtx = False
        self._pending: list[tuple[str, object, object]] = []
        self._totals: dict[str, list[float]] = {}       # scope -> [seconds, count]
        self.counters: dict[str, int] = {}
        self._dump_path: str | None = None

    def configure(self, enabled: bool, nvtx: bool = False, dump_path: str | None = None) -> None:
        self.enabled, self.nvtx = bool(enabled), bool(nvtx)
        if dump_path and self._dump_path is None:
            atexit.register(self.dump)
        self._dump_path = dump_path or self._dump_path

    @contextlib.contextmanager
    def span(self, scope: str):
        if not (self.enabled or self.nvtx):
            yield
            return
        cuda = torch.cuda.is_available() and torch.cuda.is_initialized() and not torch.cuda.is_current_stream_capturing()
        if self.nvtx and cuda:
            torch.cuda.nvtx.range_push(scope)
        if self.enabled and cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        try:
            yield
        finally:
            if self.enabled:
                if cuda:
                    e1.record()
                    self._pending.append((scope, e0, e1))
                    if len(self._pending) > 4096:
                        self._resolve()
                else:
                    tot = self._totals.setdefault(scope, [0.0, 0])
                    tot[0] += time.perf_counter() - t0
                    tot[1] += 1
            if self.nvtx and cuda:
                torch.cuda.nvtx.range_pop()

    def count(self, name: str, n: int = 1) -> None:
        if self.enabled:
            self.counters[name] = self.counters.get(name, 0) + n

    def _resolve(self) -> None:
        if not self._pending:
            return
        torch.cuda.synchronize()
        for scope, e0, e1 in self._pending:
            tot = self._totals.setdefault(scope, [0.0, 0])
            tot[0] += e0.elapsed_time(e1) / 1e3
            tot[1] += 1
        self._pending.clear()

    def summary(self) -> dict:
        self._resolve()
        out = {k: {"time_s": round(v[0], 6), "count": int(v[1]), "mean_ms": round(v[0] / max(v[1], 1) * 1e3, 4)}
               for k, v in sorted(self._totals.items(), key=lambda kv: -kv[1][0])}
        if self.counters:
            out["counters"] = dict(self.counters)
        return out

    def reset(self) -> None:
        self._pending.clear()
        self._totals.clear()
        self.counters.clear()

    def dump(self, path: str | None = None) -> None:
        path = path or self._dump_path
        if path:
            with open(path, "w") as f:
                json.dump(self.summary(), f, indent=1)


PROFILER = SpanProfiler()
span = PROFILER.span

# Per-stage spans inside a model's forward (attention / dense MLP / router / routed experts / shared expert of
# every layer, final norm + lm_head).  They are a second switch on top of the profiler itself because they
# only measure eager forwards (prefill, or decode with CUDA graphs off): under graph capture or replay no
# Python runs per stage.  ``FASTINFERENCE_PROFILE_STAGES=1`` (environment) or ``PROFILER.stages = True``.
# Reference: vllm/model_executor/models/gemma4/profiling.py:57-97 (per-stage wall-clock spans).
import os as _os

PROFILER.stages = _os.environ.get("FASTINFERENCE_PROFILE_STAGES", "0") == "1"
_NO_SPAN = contextlib.nullcontext()


def stage(scope: str):
    """``with stage("layer.attn"): ...`` - a profiler span when stage profiling is on, else a shared no-op."""
    if PROFILER.stages and (PROFILER.enabled or PROFILER.nvtx):
        return PROFILER.span(scope)
    return _NO_SPAN
