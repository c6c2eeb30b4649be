"""Runtime observer: hook interface plus an in-memory implementation with bounded histories.
Reference: vllm/engine/runtime_observer.py:11-249."""
from __future__ import annotations

import time
from collections import Counter, deque


class RuntimeObserver:
    def on_request_added(self, request_id: str, prompt_len: int) -> None: ...
    def on_request_admitted(self, request_id: str, queue_wait_s: float) -> None: ...
    def on_request_rejected(self, request_id: str, reason: str) -> None: ...
    def on_request_finished(self, request_id: str, reason: str, n_tokens: int) -> None: ...
    def on_request_aborted(self, request_id: str) -> None: ...
    def on_first_token(self, request_id: str, ttft_s: float) -> None: ...
    def on_prefix_cache_event(self, kind: str, tokens: int = 0) -> None: ...
    def on_step_started(self, plan) -> None: ...
    def on_prefill_executed(self, n_seqs: int, n_tokens: int, seconds: float) -> None: ...
    def on_decode_executed(self, n_seqs: int, seconds: float) -> None: ...
    def on_background_error(self, exc: BaseException) -> None: ...
    def on_model_surface(self, surface: dict) -> None: ...
    def on_rank_event(self, kind: str, rank: int) -> None: ...
    def on_model_event(self, event: str, **payload) -> None: ...       # events of a model-owned data plane
    def stats(self) -> dict: return {}
    def reset(self) -> None: ...


class InMemoryRuntimeObserver(RuntimeObserver):
    def __init__(self, history: int = 512):
        self.history = history
        self.reset()

    def reset(self) -> None:
        self.counters: Counter = Counter()
        self.ttft = deque(maxlen=self.history)
        self.queue_wait = deque(maxlen=self.history)
        self.prefill_steps = deque(maxlen=self.history)
        self.decode_steps = deque(maxlen=self.history)
        self.reject_reasons: Counter = Counter()
        self.finish_reasons: Counter = Counter()
        self.last_error: str | None = None
        self.model_surface: dict = {}
        self.model_events: Counter = Counter()
        self.last_model_event: dict = {}
        self.started = time.monotonic()

    def on_request_added(self, request_id, prompt_len):
        self.counters["requests_added"] += 1
        self.counters["prompt_tokens"] += prompt_len

    def on_request_admitted(self, request_id, queue_wait_s):
        self.counters["requests_admitted"] += 1
        self.queue_wait.append(queue_wait_s)

    def on_request_rejected(self, request_id, reason):
        self.counters["requests_rejected"] += 1
        self.reject_reasons[reason] += 1

    def on_request_finished(self, request_id, reason, n_tokens):
        self.counters["requests_finished"] += 1
        self.counters["generated_tokens"] += n_tokens
        self.finish_reasons[reason] += 1

    def on_request_aborted(self, request_id):
        self.counters["requests_aborted"] += 1

    def on_first_token(self, request_id, ttft_s):
        self.ttft.append(ttft_s)

    def on_prefix_cache_event(self, kind, tokens=0):
        self.counters[f"prefix_cache_{kind}"] += 1
        self.counters["prefix_cache_tokens"] += tokens

    def on_step_started(self, plan):
        self.counters["steps"] += 1
        if plan.metrics.get("starvation_override"):
            self.counters["starvation_overrides"] += 1
        if plan.fast_path:
            self.counters["fast_path_steps"] += 1

    def on_prefill_executed(self, n_seqs, n_tokens, seconds):
        self.counters["prefill_tokens"] += n_tokens
        self.prefill_steps.append((n_seqs, n_tokens, seconds))

    def on_decode_executed(self, n_seqs, seconds):
        self.counters["decode_tokens"] += n_seqs
        self.decode_steps.append((n_seqs, seconds))

    def on_background_error(self, exc):
        self.counters["background_errors"] += 1
        self.last_error = repr(exc)

    def on_model_surface(self, surface):
        self.model_surface = dict(surface)

    def on_rank_event(self, kind, rank):
        self.counters[f"rank_{kind}"] += 1

    @staticmethod
    def _pct(values, q):
        if not values:
            return None
        s = sorted(values)
        return s[min(len(s) - 1, int(q * len(s)))]

    def on_model_event(self, event, **payload):
        self.model_events[event] += 1
        self.last_model_event[event] = payload

    def stats(self) -> dict:
        dec = list(self.decode_steps)
        dec_time = sum(s for _, s in dec)
        return {
            "counters": dict(self.counters), "reject_reasons": dict(self.reject_reasons),
            "finish_reasons": dict(self.finish_reasons),
            "ttft_p50_s": self._pct(list(self.ttft), 0.5), "ttft_p95_s": self._pct(list(self.ttft), 0.95),
            "queue_wait_p50_s": self._pct(list(self.queue_wait), 0.5),
            "decode_tokens_per_s": (sum(n for n, _ in dec) / dec_time) if dec_time > 0 else None,
            "last_error": self.last_error, "model_surface": self.model_surface,
            "model_events": {"counts": dict(self.model_events), "last": dict(self.last_model_event)},
            "uptime_s": time.monotonic() - self.started,
        }
