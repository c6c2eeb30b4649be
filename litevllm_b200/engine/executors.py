"""Prefill and decode executors: build the batch, run the model, return logits (or tokens).

The decode executor captures one CUDA graph per batch-size bucket (inputs live in persistent
buffers owned by the batch builder) and replays it on later steps; the reference launches every
kernel from Python each step (vllm/engine/decode_executor.py:29-70,
vllm/engine/prefill_executor.py:21-70).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..utils.profiling import span

from .. import ops
from .input_batch import ForwardBatch, InputBatchBuilder
from .request_state import RequestState
from .step_plan import PrefillItem


@dataclass
class LogitsResult:
    logits: torch.Tensor            # [num_seqs, vocab] float32
    request_ids: list[str]


@dataclass
class TokenPrefillResult:
    token_ids: list[int]
    request_ids: list[str]


@dataclass
class TokenDecodeResult:
    token_ids: list[int]
    request_ids: list[str]


class PrefillExecutor:
    def __init__(self, model, kv_cache, builder: InputBatchBuilder, multimodal=None):
        self.model, self.kv_cache, self.builder, self.multimodal = model, kv_cache, builder, multimodal

    @torch.inference_mode()
    def execute(self, items: list[PrefillItem], states: dict[str, RequestState], lora_mapping=None) -> LogitsResult:
        batch = self.builder.build_prefill(items, states)
        batch.lora_mapping = lora_mapping
        embeds = None
        if self.multimodal is not None:
            embeds = self.multimodal.embed_for_prefill(self.model, batch, items, states)
        if hasattr(self.model, "prepare_batch"):
            self.model.prepare_batch(batch, states)
        if hasattr(self.model, "prepare_prefill"):      # prefill-only hook (does not make the decode step stateful)
            self.model.prepare_prefill(batch, items, states)
        with span("prefill_forward"):
            logits = self.model(batch, self.kv_cache, inputs_embeds=embeds)
        if hasattr(self.model, "finish_batch"):
            self.model.finish_batch(batch, states)
        return LogitsResult(logits, batch.request_ids)


class DecodeExecutor:
    def __init__(self, model, kv_cache, builder: InputBatchBuilder, use_cuda_graph: bool = True):
        self.model, self.kv_cache, self.builder = model, kv_cache, builder
        self.use_cuda_graph = use_cuda_graph and builder.device.type == "cuda" and \
            getattr(model, "supports_cuda_graph", True)
        self._graphs: dict[int, tuple] = {}
        self._pool = None
        self.graph_replays = 0
        self.eager_steps = 0
        self.launches_per_graph: dict[int, int] = {}

    def _run(self, batch: ForwardBatch) -> torch.Tensor:
        batch.extras.pop("_selected_blocks", None)      # per-step product of the selective-attention kernel
        return self.model(batch, self.kv_cache)

    def _step_body(self, batch: ForwardBatch, greedy_only: bool = False) -> torch.Tensor:
        """What one captured decode step consists of: gather the block-table rows of the batch's
        slots, run the model, and leave the greedy token of every row in the input-id buffer (the
        next pipelined step reads its ids from there; other callers overwrite the buffer anyway).
        Keeping all three inside the graph leaves one host-to-device and one device-to-host copy
        per step outside it.  ``greedy_only``: nobody will look at the logits, so a model whose
        lm_head is sharded over the vocabulary may write the tokens itself from its local slice
        (vocabulary-parallel arg-max) instead of gathering full logits."""
        d = self.builder._decode_buffers(batch.num_seqs)
        ops.gather_rows_i32(self.builder.kv.block_tables, d["meta"][3], d["block_tables"])
        batch.extras.pop("greedy_done", None)
        if greedy_only:
            batch.extras["greedy_out"] = d["ids"]
        else:
            batch.extras.pop("greedy_out", None)
        logits = self._run(batch)
        if not batch.extras.pop("greedy_done", False):
            ops.argmax(logits, out=d["ids"])
        return logits

    @torch.inference_mode()
    def execute_batch(self, reqs: list[RequestState], states: dict[str, RequestState] | None = None,
                      device_tokens: torch.Tensor | None = None, lora_mapping=None) -> LogitsResult:
        batch = self.builder.build_decode(reqs, device_tokens)
        batch.lora_mapping = lora_mapping
        stateful = hasattr(self.model, "prepare_batch")
        if stateful:
            self.model.prepare_batch(batch, states or {r.request_id: r for r in reqs})
        if not self.use_cuda_graph or lora_mapping is not None or stateful:
            self.eager_steps += 1
            with span("decode_forward_eager"):
                logits = self._run(batch)
            if stateful:
                self.model.finish_batch(batch, states or {r.request_id: r for r in reqs})
            return LogitsResult(logits, batch.request_ids)
        key = (batch.num_seqs, False)
        entry = self._graphs.get(key)
        if entry is None:
            entry = self._capture(batch)
            self._graphs[key] = entry
        graph, out, max_kv_cap = entry
        if batch.max_kv_len > max_kv_cap:
            # attention split count was chosen for a shorter context: recapture
            entry = self._capture(batch)
            self._graphs[key] = entry
            graph, out, max_kv_cap = entry
        with span("decode_graph_replay"):
            graph.replay()
        self.graph_replays += 1
        return LogitsResult(out, batch.request_ids)

    def _capture(self, batch: ForwardBatch, greedy_only: bool = False):
        # graphs are captured for the full context so one graph serves the whole request lifetime
        full_ctx = self.builder.kv.blocks_per_seq * self.builder.kv.block_size
        saved = batch.max_kv_len
        batch.max_kv_len = full_ctx
        # warm up outside capture (lazy allocations, scratch growth, kernel attribute setup)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        ids_saved = batch.input_ids.clone()
        with torch.cuda.stream(side):
            for _ in range(2):
                self._step_body(batch, greedy_only)
                batch.input_ids.copy_(ids_saved)      # the body leaves the greedy tokens in the id buffer
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        n0 = ops.launch_count()
        with torch.cuda.graph(graph, pool=self._pool):
            out = self._step_body(batch, greedy_only)
        self.launches_per_graph[batch.num_seqs] = ops.launch_count() - n0
        if self._pool is None:
            self._pool = graph.pool()
        batch.max_kv_len = saved
        ops.check_status(self.builder.device)
        return graph, out, full_ctx

    @torch.inference_mode()
    def replay_or_capture(self, bucket: int, reqs: list[RequestState], max_kv_len: int) -> torch.Tensor:
        """Run the decode forward on the persistent bucket buffers (already filled by the caller)
        and return the logits tensor (the pipelined decode only uses the greedy tokens the step left in
        the id buffer; under a vocabulary-sharded lm_head the logits are this rank's slice)."""
        d = self.builder._decode_buffers(bucket)
        batch = ForwardBatch(
            input_ids=d["ids"], positions=d["meta"][0], slot_mapping=d["meta"][1], block_tables=d["block_tables"],
            seq_lens=d["meta"][2], cu_q=None, logits_indices=None, num_seqs=bucket, num_tokens=bucket, max_q_len=1,
            max_kv_len=max_kv_len, is_decode=True, config=self.builder.cfg,
            request_ids=[st.request_id for st in reqs],
            extras={"num_real": len(reqs), "bucket": bucket, "slot_ids": d["meta"][3]})
        if not self.use_cuda_graph:
            self.eager_steps += 1
            return self._step_body(batch, greedy_only=True)
        key = (bucket, True)
        entry = self._graphs.get(key)
        if entry is None:
            entry = self._capture(batch, greedy_only=True)
            self._graphs[key] = entry
        with span("decode_graph_replay"):
            entry[0].replay()
        self.graph_replays += 1
        return entry[1]

    def execute_sync_fast(self, st: RequestState, device_tokens=None) -> LogitsResult:
        return self.execute_batch([st], device_tokens=device_tokens)
