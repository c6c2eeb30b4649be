"""Token-returning executors for the model-owned DeepSeek-V4-Flash data plane: the engine hands over plan
items and request states, the model consumes token ids and returns token ids (greedy), and the backend skips
its sampler for these results.  Reference: vllm/engine/deepseek_v4_flash_executors.py:12-89."""
from __future__ import annotations

import time

import torch

from ...engine.executors import TokenDecodeResult, TokenPrefillResult
from ...utils.profiling import span


def _record(observer, event: str, **payload) -> None:
    hook = getattr(observer, "on_model_event", None)
    if callable(hook):
        hook(event, **payload)


class V4FlashPrefillExecutor:
    def __init__(self, model, observer=None):
        self.model, self.observer = model, observer

    @torch.inference_mode()
    def execute(self, items, states, lora_mapping=None) -> TokenPrefillResult:
        tokens, rids = [], []
        with span("prefill_forward"):
            for it in items:
                st = states[it.request_id]
                final = it.end >= st.prompt_len
                fresh = it.request_id not in self.model.requests or it.start == 0
                tok = self.model.prefill_request(it.request_id, st.prompt_token_ids[it.start:it.end], it.start, final)
                tokens.append(-1 if tok is None else tok)
                rids.append(it.request_id)
                if fresh:         # the request's row pools now exist
                    _record(self.observer, "rows_allocated", request_id=it.request_id, token_count=it.end,
                            **self.model.kv_stats())
        return TokenPrefillResult(tokens, rids)


class V4FlashDecodeExecutor:
    """No ``replay_or_capture``: the pipelined graph decode is skipped for this model."""

    def __init__(self, model, observer=None):
        self.model, self.observer = model, observer
        self.graph_replays = 0
        self.eager_steps = 0
        self.launches_per_graph: dict[int, int] = {}

    @torch.inference_mode()
    def execute_batch(self, reqs, states=None, device_tokens=None, lora_mapping=None) -> TokenDecodeResult:
        self.eager_steps += 1
        t0 = time.perf_counter()
        with span("decode_forward_eager"):
            toks = self.model.decode_tokens_batch([st.request_id for st in reqs], [st.last_token() for st in reqs])
        _record(self.observer, "decode_batch", batch_size=len(reqs), latency_ms=(time.perf_counter() - t0) * 1e3)
        return TokenDecodeResult(toks, [st.request_id for st in reqs])

    def execute_sync_fast(self, st, device_tokens=None) -> TokenDecodeResult:
        return self.execute_batch([st])
