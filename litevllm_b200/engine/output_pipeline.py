"""Turns sampled tokens into ``RequestOutput`` objects and decides when a request is finished.

Finish rules: EOS (once ``min_tokens`` is reached and ``ignore_eos`` is off) -> "stop"; stop strings
-> "stop"; ``max_tokens`` or the context limit -> "length"; a structured-output constraint may end
the request itself.  Intermediate outputs carry a lazy text decoder; the final output is decoded
eagerly.  Reference: vllm/engine/output_pipeline.py:11-122, vllm/engine/output_processor.py:8-99.
"""
from __future__ import annotations

import time

from ..outputs import CompletionOutput, RequestOutput
from .request_state import RequestState


class OutputProcessor:
    """Per-model hook points (identity by default)."""

    def on_token(self, st: RequestState, token_id: int) -> int:
        return token_id

    def postprocess_text(self, st: RequestState, text: str) -> str:
        return text


class GenerationPolicies:
    def __init__(self, output_processor: OutputProcessor | None = None, early_stop=None):
        self.output_processor = output_processor or OutputProcessor()
        self.early_stop = early_stop


class OutputPipeline:
    def __init__(self, tokenizer, max_model_len: int, policies: GenerationPolicies | None = None):
        self.tokenizer = tokenizer
        self.max_model_len = max_model_len
        self.policies = policies or GenerationPolicies()

    def _decode(self, st: RequestState):
        skip = st.sampling_params.skip_special_tokens
        tok = self.tokenizer

        def fn(ids):
            if tok is None or not st.sampling_params.detokenize:
                return ""
            return tok.decode(ids, skip_special_tokens=skip)
        return fn

    def check_finish(self, st: RequestState, token_id: int) -> str | None:
        sp = st.sampling_params
        n = len(st.generated_ids)
        if (token_id in st.eos_token_ids and not sp.ignore_eos and n >= sp.min_tokens):
            return "stop"
        c = st.structured_output_constraint
        if c is not None and c.should_finish():
            return "stop"
        if sp.max_tokens is not None and n >= sp.max_tokens:
            return "length"
        if st.prompt_len + n >= self.max_model_len:
            return "length"
        if self.policies.early_stop is not None and self.policies.early_stop(st):
            return "stop"
        return None

    def finalize_step(self, st: RequestState, token_id: int) -> RequestOutput:
        """Append one sampled token and build the output for this step."""
        token_id = self.policies.output_processor.on_token(st, int(token_id))
        st.generated_ids.append(token_id)
        if st.first_token_time is None:
            st.first_token_time = time.monotonic()
        c = st.structured_output_constraint
        if c is not None:
            c.on_token(token_id)
        reason = self.check_finish(st, token_id)
        text = None
        if reason is None and st.sampling_params.stop and st.sampling_params.detokenize:
            text = self._decode(st)(st.generated_ids)
            for s in st.sampling_params.stop:
                k = text.find(s)
                if k >= 0:
                    reason = "stop"
                    text = text[: k + (len(s) if st.sampling_params.include_stop_str_in_output else 0)]
                    break
            if reason is None:
                text = None
        return self.make_output(st, reason, text)

    def make_output(self, st: RequestState, reason: str | None, text: str | None = None) -> RequestOutput:
        ids = list(st.generated_ids)
        if reason is not None:
            st.finished, st.finish_reason, st.finished_time = True, reason, time.monotonic()
            if text is None:
                text = self._decode(st)(ids)
            text = self.policies.output_processor.postprocess_text(st, text)
        comp = CompletionOutput(index=0, token_ids=ids, text=text, decode=self._decode(st),
                                cumulative_logprob=0.0, finish_reason=reason)
        metrics = {}
        if st.first_token_time is not None and st.admitted_time is not None:
            metrics["ttft_s"] = st.first_token_time - st.arrival_time
        return RequestOutput(request_id=st.request_id, prompt=st.prompt, prompt_token_ids=st.prompt_token_ids,
                             outputs=[comp], finished=reason is not None, finish_reason=reason, metrics=metrics)
