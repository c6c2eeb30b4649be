"""Execution backend of one GPU rank: grows KV block tables, runs the executors, samples, finalises
outputs and releases finished requests.

Greedy fast path: for requests whose only stop condition is ``max_tokens`` the sampled token stays
on the device and feeds the next step directly; the host copies all tokens once at the end.
Prefix cache: when enabled, whole-block prompt prefixes (KV blocks + last-position logits) are kept
in an LRU and materialised into new requests' blocks.
Reference: vllm/engine/backend/lite_single_gpu.py:66-569.
"""
from __future__ import annotations

import time

import torch

from .errors import ExecutionStepError
from .executors import TokenDecodeResult, TokenPrefillResult
from .request_state import RequestState
from .sampling_driver import SamplingDriver
from .step_plan import StepPlan


class LiteGpuBackend:
    def __init__(self, scheduler, kv_manager, prefill_executor, decode_executor, sampling_driver: SamplingDriver,
                 output_pipeline, observer, backend_policy, prefix_cache=None, lora_registry=None,
                 on_release=None):
        self.scheduler = scheduler
        self.kv = kv_manager
        self.prefill_executor = prefill_executor
        self.decode_executor = decode_executor
        self.sampling = sampling_driver
        self.outputs = output_pipeline
        self.observer = observer
        self.policy = backend_policy
        self.prefix_cache = prefix_cache
        self.lora_registry = lora_registry
        self.on_release = on_release
        self.greedy_device_steps = 0
        self.pipeline = None
        self.pipelined_steps = 0
        self.async_decode = getattr(backend_policy, "async_decode", True)

    # ------------------------------------------------------------------ KV growth
    def ensure_kv_blocks(self, plan: StepPlan) -> None:
        for it in plan.prefills:
            self.kv.ensure_blocks(it.request_id, it.end)
        for rid in plan.decodes:
            st = self.scheduler.requests[rid]
            self.kv.ensure_blocks(rid, st.seq_len + 1)

    def register_admitted(self, st: RequestState) -> None:
        self.kv.register(st.request_id, st.slot_idx)

    # ------------------------------------------------------------------ prefix cache
    def maybe_apply_prefix_cache(self, st: RequestState) -> None:
        pc = self.prefix_cache
        if pc is None or not pc.enabled or st.slot_idx < 0:
            return
        hit = pc.lookup(st)
        if hit is None:
            self.observer.on_prefix_cache_event("miss")
            return
        n_tokens = min(hit.num_tokens, (st.prompt_len - 1) // self.kv.block_size * self.kv.block_size) \
            if hit.num_tokens >= st.prompt_len and hit.logits is None else hit.num_tokens
        if n_tokens <= 0:
            return
        self.kv.materialize_prefix(st.request_id, hit.blocks, n_tokens // self.kv.block_size)
        st.seq_len = n_tokens
        st.prefix_cache_hit_tokens = n_tokens
        if n_tokens >= st.prompt_len and hit.logits is not None:
            st.cached_first_logits = hit.logits
        self.observer.on_prefix_cache_event("hit", n_tokens)

    def _maybe_store_prefix(self, st: RequestState, logits_row) -> None:
        pc = self.prefix_cache
        if pc is None or not pc.enabled:
            return
        n = st.prompt_len // self.kv.block_size * self.kv.block_size
        if n <= 0 or pc.contains(st, n):
            return
        blocks = self.kv.capture_prefix(st.request_id, n)
        if blocks is not None:
            keep_logits = logits_row.clone() if (logits_row is not None and n == st.prompt_len) else None
            pc.store(st, n, blocks, keep_logits)
            self.observer.on_prefix_cache_event("store", n)

    # ------------------------------------------------------------------ steps
    def run_prefills(self, plan: StepPlan) -> list:
        if not plan.prefills:
            return []
        states = self.scheduler.requests
        outs = self.drain_pipeline()
        # exact prefix hits sample their first token from the cached logits without a forward pass
        items = []
        for it in plan.prefills:
            st = states[it.request_id]
            if st.cached_first_logits is not None and st.seq_len >= st.prompt_len:
                tok = self.sampling.sample_batch_tokens(st.cached_first_logits[None].float(), [st])[0]
                st.cached_first_logits = None
                st.is_prefill = False
                outs.append(self._process_completion(st, tok))
            else:
                items.append(it)
        if not items:
            return outs
        t0 = time.perf_counter()
        try:
            lora_map = self.lora_registry.mapping_for_prefill(items, states) if self.lora_registry else None
            res = self.prefill_executor.execute(items, states, lora_mapping=lora_map)
        except Exception as e:
            raise ExecutionStepError(f"prefill step failed: {e!r}") from e
        done_reqs, done_rows = [], []
        for row, it in enumerate(items):
            st = states[it.request_id]
            st.seq_len = it.end
            if st.seq_len >= st.prompt_len:
                st.is_prefill = False
                done_reqs.append(st)
                done_rows.append(row)
        if done_reqs:
            if isinstance(res, TokenPrefillResult):
                tokens = [res.token_ids[r] for r in done_rows]
            else:
                rows = res.logits if len(done_rows) == len(items) else res.logits[done_rows]
                for st, r in zip(done_reqs, done_rows):
                    self._maybe_store_prefix(st, res.logits[r])
                tokens = self._sample(rows, done_reqs)
            for st, tok in zip(done_reqs, tokens):
                outs.append(self._process_completion(st, tok))
        self.observer.on_prefill_executed(len(items), sum(i.chunk_len for i in items), time.perf_counter() - t0)
        return outs

    # ------------------------------------------------------------------ pipelined decode
    def _pipeline_ok(self, reqs, plan: StepPlan) -> bool:
        ex = self.decode_executor
        if not self.async_decode or not hasattr(ex, "replay_or_capture") or ex.builder.device.type != "cuda":
            return False
        if hasattr(ex.model, "prepare_batch") or plan.prefills:
            return False
        from .decode_pipeline import DecodePipeline
        return all(DecodePipeline.eligible(st) for st in reqs)

    def _consume_tokens(self, reqs, tokens, outs: list) -> bool:
        """Feed one step's tokens to the output pipeline; returns True if any request finished."""
        any_finished = False
        for st, tok in zip(reqs, tokens):
            if st.finished or st.request_id not in self.scheduler.requests:
                continue
            out = self._process_completion(st, int(tok))
            if out is not None:
                outs.append(out)
                any_finished |= out.finished
        return any_finished

    def drain_pipeline(self) -> list:
        """Collect every in-flight step (used when the request set is about to change)."""
        outs: list = []
        pipe = self.pipeline
        if pipe is None or not pipe.active:
            return outs
        reqs = list(pipe.reqs)
        while pipe.inflight:
            self._consume_tokens(reqs, pipe.collect_oldest(), outs)
        pipe.stop()
        return outs

    def _run_decodes_pipelined(self, reqs) -> list:
        from .decode_pipeline import DecodePipeline
        if self.pipeline is None:
            self.pipeline = DecodePipeline(self.decode_executor, self.decode_executor.builder, self.kv)
        pipe = self.pipeline
        outs: list = []
        key = tuple(st.request_id for st in reqs)
        if pipe.active and pipe.key != key:
            outs += self.drain_pipeline()
            reqs = [st for st in reqs if not st.finished and st.request_id in self.scheduler.requests]
            if not reqs:
                return outs
        if not pipe.active:
            for st in reqs:
                self._flush_pending(st)
            pipe.start(reqs)
        if pipe.can_launch():
            pipe.launch()
            self.pipelined_steps += 1
            # keep one step in flight: look at the step before the one just launched
            if len(pipe.inflight) > 1:
                if self._consume_tokens(pipe.reqs, pipe.collect_oldest(), outs):
                    outs += self.drain_pipeline()
        else:
            outs += self.drain_pipeline()
        return outs

    def run_decodes(self, plan: StepPlan) -> list:
        if not plan.decodes:
            if self.pipeline is not None and self.pipeline.active:
                return self.drain_pipeline()
            return []
        states = self.scheduler.requests
        reqs = [states[r] for r in plan.decodes if r in states and not states[r].finished]
        if not reqs:
            return []
        if self._pipeline_ok(reqs, plan):
            t0 = time.perf_counter()
            outs = self._run_decodes_pipelined(reqs)
            self.observer.on_decode_executed(len(reqs), time.perf_counter() - t0)
            return outs
        if self.pipeline is not None and self.pipeline.active:
            pre = self.drain_pipeline()
            reqs = [st for st in reqs if not st.finished and st.request_id in states]
            if not reqs:
                return pre
            return pre + self._run_decodes_sync(reqs, states)
        return self._run_decodes_sync(reqs, states)

    def _run_decodes_sync(self, reqs, states) -> list:
        t0 = time.perf_counter()
        try:
            on_device = all(st.last_token_tensor is not None for st in reqs)
            dev_tokens = torch.stack([st.last_token_tensor for st in reqs]) if on_device else None
            if not on_device:
                for st in reqs:
                    self._flush_pending(st)
            lora_map = self.lora_registry.mapping_for_decode(reqs) if self.lora_registry else None
            res = self.decode_executor.execute_batch(reqs, states, device_tokens=dev_tokens, lora_mapping=lora_map)
        except Exception as e:
            raise ExecutionStepError(f"decode step failed: {e!r}") from e
        for st in reqs:
            st.seq_len += 1
        if isinstance(res, TokenDecodeResult):
            tokens = res.token_ids
        else:
            tokens = self._sample(res.logits, reqs)
        outs = [self._process_completion(st, tok) for st, tok in zip(reqs, tokens)]
        self.observer.on_decode_executed(len(reqs), time.perf_counter() - t0)
        return [o for o in outs if o is not None]

    def decode_step_sync(self, request_id: str) -> list:
        return self.run_decodes(StepPlan(decodes=[request_id], fast_path=True))

    # ------------------------------------------------------------------ sampling + completion
    def _sample(self, logits, reqs: list[RequestState]):
        """Returns a list with one entry per request: an int, or a 0-d device tensor for requests
        that may keep their tokens on the device."""
        keep = [self.sampling.can_stay_on_device(st, self.policy) for st in reqs]
        dev = self.sampling.sample_device(logits, reqs)
        if all(keep) and dev.is_cuda:
            self.greedy_device_steps += 1
            return list(dev.unbind(0))
        return dev.tolist()

    def _flush_pending(self, st: RequestState) -> None:
        if st.pending_token_tensors:
            toks = torch.stack(st.pending_token_tensors).tolist()
            st.pending_token_tensors.clear()
            st.generated_ids.extend(int(t) for t in toks)
        st.last_token_tensor = None

    def _process_completion(self, st: RequestState, token):
        if isinstance(token, torch.Tensor):
            # device-resident token: only max_tokens / context can end this request
            st.pending_token_tensors.append(token)
            st.last_token_tensor = token
            if st.first_token_time is None:
                st.first_token_time = time.monotonic()
                self.observer.on_first_token(st.request_id, st.first_token_time - st.arrival_time)
            n = st.num_generated
            sp = st.sampling_params
            if (sp.max_tokens is not None and n >= sp.max_tokens) or st.prompt_len + n >= self.outputs.max_model_len:
                self._flush_pending(st)
                out = self.outputs.make_output(st, "length")
                self._finish(st, out)
                return out
            return None
        first = st.first_token_time is None
        out = self.outputs.finalize_step(st, int(token))
        if first:
            self.observer.on_first_token(st.request_id, st.first_token_time - st.arrival_time)
        if out.finished:
            self._finish(st, out)
        else:
            self.scheduler.publish_output(st.request_id, out)
        return out

    def _finish(self, st: RequestState, out) -> None:
        # terminal publication precedes resource release
        self.scheduler.publish_output(st.request_id, out)
        self.observer.on_request_finished(st.request_id, out.finish_reason or "", len(st.generated_ids))
        self.release_request(st.request_id)

    def release_request(self, request_id: str) -> None:
        pipe = self.pipeline
        if pipe is not None and pipe.active and request_id in pipe.key and pipe.inflight:
            # an in-flight step still writes this request's KV blocks: let it finish first
            torch.cuda.current_stream().synchronize()
        self.kv.release(request_id)
        st = self.scheduler.release(request_id)
        if st is not None and self.on_release is not None:
            self.on_release(st)

    def stats(self) -> dict:
        return {"kv": self.kv.stats(), "greedy_device_steps": self.greedy_device_steps,
                "pipelined_decode_steps": self.pipelined_steps,
                "graph_replays": getattr(self.decode_executor, "graph_replays", 0),
                "eager_decode_steps": getattr(self.decode_executor, "eager_steps", 0),
                "prefix_cache": self.prefix_cache.stats() if self.prefix_cache else {"enabled": False},
                "gpu_greedy_sampling": self.policy.gpu_greedy_sampling}
