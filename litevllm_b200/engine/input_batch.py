"""Batch metadata for one forward pass over a flattened varlen token stream.

All per-step integers are assembled in ONE pinned host buffer and reach the device in a single
asynchronous copy (ids as int64, everything else int32), instead of several small writes per
request.  Decode batches are padded to a bucket size so that CUDA graphs captured per bucket can be
replayed; padded rows have ``seq_len = 0`` and ``slot = -1`` and are ignored by every kernel.
Reference: vllm/engine/input_batch_builder.py:38-479 (rectangular [B, T] batches, per-token
metadata expansion for prefill, Triton slot-mapping kernel).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch

from ..config.inference_config import LiteInferenceConfig
from .request_state import RequestState
from .step_plan import PrefillItem


@dataclass
class ForwardBatch:
    input_ids: torch.Tensor          # [T] int64
    positions: torch.Tensor          # [T] int32 (or [3, T] for multimodal rotary)
    slot_mapping: torch.Tensor       # [T] int32, -1 = do not write
    block_tables: torch.Tensor       # [B, blocks_per_seq] int32
    seq_lens: torch.Tensor           # [B] int32: KV length after this step
    cu_q: torch.Tensor | None        # [B+1] int32 (prefill)
    logits_indices: torch.Tensor | None   # [B] int64 rows of the last token of each sequence
    num_seqs: int
    num_tokens: int
    max_q_len: int
    max_kv_len: int
    is_decode: bool
    config: LiteInferenceConfig
    request_ids: list[str] = field(default_factory=list)
    lora_mapping: Any = None
    multimodal: Any = None
    seq_lens_cpu: list[int] = field(default_factory=list)
    q_lens_cpu: list[int] = field(default_factory=list)
    extras: dict = field(default_factory=dict)   # model-specific carries (linear-attention state, ...)

    def attention_tables(self, window: int = 0):
        """``(block_tables, seq_lens)`` an attention layer should read.  With selective attention on
        (``kv_select_ratio`` > 0) a decode step's global-attention layers (no sliding window) get the compact
        tables of the kept blocks; they are built once per step, by one kernel, the first time a layer asks."""
        cfg = self.config
        if not self.is_decode or window or getattr(cfg, "kv_select_ratio", 0.0) <= 0.0:
            return self.block_tables, self.seq_lens
        sel = self.extras.get("_selected_blocks")
        if sel is None:
            from .. import ops
            stride = max(1, int(1.0 / cfg.kv_select_ratio))
            sel = ops.select_blocks(self.block_tables, self.seq_lens, cfg.block_size, stride, cfg.kv_select_min_blocks)
            self.extras["_selected_blocks"] = sel
        return sel


def decode_buckets(max_active: int) -> list[int]:
    out, b = [], 1
    while b < max_active:
        out.append(b)
        b *= 2
    out.append(max_active)
    return out


class InputBatchBuilder:
    def __init__(self, kv_manager, max_active: int, max_step_tokens: int, device: torch.device,
                 inf_config: LiteInferenceConfig):
        self.kv = kv_manager
        self.device = device
        self.cfg = inf_config
        self.max_active = max_active
        self.bs = kv_manager.block_size
        self.buckets = decode_buckets(max_active)
        pin = device.type == "cuda"
        cap = max(max_step_tokens, max_active) + 8
        self._cap = cap
        # host staging: ids (int64) then int32 meta [positions | slots | token_seq] + per-seq arrays
        self._h_ids = torch.zeros(cap, dtype=torch.int64, pin_memory=pin)
        self._h_meta = torch.zeros(2 * cap + 4 * (max_active + 1), dtype=torch.int32, pin_memory=pin)
        self._d_ids = torch.zeros(cap, dtype=torch.int64, device=device)
        self._d_meta = torch.zeros_like(self._h_meta, device=device)
        # persistent decode inputs per bucket (CUDA-graph inputs): [ids int64 | pos, slots, seq_lens, slot_ids]
        self._dec: dict[int, dict] = {}

    # ------------------------------------------------------------------ helpers
    def _slots_for(self, blocks: list[int], start: int, n: int) -> np.ndarray:
        pos = np.arange(start, start + n, dtype=np.int64)
        blk = np.asarray(blocks, dtype=np.int64)[pos // self.bs]
        return (blk * self.bs + pos % self.bs).astype(np.int32)

    def bucket_for(self, n: int) -> int:
        for b in self.buckets:
            if b >= n:
                return b
        return self.buckets[-1]

    # ------------------------------------------------------------------ prefill
    def build_prefill(self, items: list[PrefillItem], states: dict[str, RequestState]) -> ForwardBatch:
        B = len(items)
        T = sum(it.chunk_len for it in items)
        if T > self._cap:
            raise ValueError(f"prefill step of {T} tokens exceeds the staging capacity {self._cap}")
        ids = self._h_ids.numpy()
        meta = self._h_meta.numpy()
        pos_h, slot_h = meta[:T], meta[T:2 * T]
        base = 2 * T
        cu_h = meta[base:base + B + 1]
        sl_h = meta[base + B + 1:base + 2 * B + 1]
        sid_h = meta[base + 2 * B + 1:base + 3 * B + 1]
        off = 0
        cu_h[0] = 0
        q_lens, kv_lens = [], []
        for i, it in enumerate(items):
            st = states[it.request_id]
            n = it.chunk_len
            ids[off:off + n] = st.prompt_token_ids[it.start:it.end]
            pos_h[off:off + n] = np.arange(it.start, it.end, dtype=np.int32)
            slot_h[off:off + n] = self._slots_for(self.kv.blocks_of(it.request_id), it.start, n)
            off += n
            cu_h[i + 1] = off
            sl_h[i] = it.end
            sid_h[i] = st.slot_idx
            q_lens.append(n)
            kv_lens.append(it.end)
        n_meta = base + 3 * B + 1
        self._d_ids[:T].copy_(self._h_ids[:T], non_blocking=True)
        self._d_meta[:n_meta].copy_(self._h_meta[:n_meta], non_blocking=True)
        dm = self._d_meta
        cu = dm[base:base + B + 1]
        slot_ids = dm[base + 2 * B + 1:base + 3 * B + 1]
        self.kv.flush()
        block_tables = self.kv.block_tables.index_select(0, slot_ids.long())
        return ForwardBatch(
            input_ids=self._d_ids[:T], positions=dm[:T], slot_mapping=dm[T:2 * T],
            block_tables=block_tables, seq_lens=dm[base + B + 1:base + 2 * B + 1], cu_q=cu,
            logits_indices=(cu[1:] - 1).long(), num_seqs=B, num_tokens=T, max_q_len=max(q_lens),
            max_kv_len=max(kv_lens), is_decode=False, config=self.cfg,
            request_ids=[it.request_id for it in items], seq_lens_cpu=kv_lens, q_lens_cpu=q_lens,
            extras={"slot_ids": slot_ids})

    # ------------------------------------------------------------------ decode
    def _decode_buffers(self, bucket: int) -> dict:
        d = self._dec.get(bucket)
        if d is None:
            pin = self.device.type == "cuda"
            d = {
                "h_ids": torch.zeros(bucket, dtype=torch.int64, pin_memory=pin),
                "h_meta": torch.zeros(4, bucket, dtype=torch.int32, pin_memory=pin),
                "ids": torch.zeros(bucket, dtype=torch.int64, device=self.device),
                "meta": torch.zeros(4, bucket, dtype=torch.int32, device=self.device),
                "block_tables": torch.zeros(bucket, self.kv.blocks_per_seq, dtype=torch.int32, device=self.device),
            }
            self._dec[bucket] = d
        return d

    def build_decode(self, reqs: list[RequestState], device_tokens: torch.Tensor | None = None) -> ForwardBatch:
        """One new token per request.  ``device_tokens`` (int64 [n]) supplies the input ids from the
        device (greedy fast path); otherwise they come from ``generated_ids``."""
        n = len(reqs)
        bucket = self.bucket_for(n)
        d = self._decode_buffers(bucket)
        hm = d["h_meta"].numpy()
        hi = d["h_ids"].numpy()
        hm[0, n:] = 0
        hm[1, n:] = -1
        hm[2, n:] = 0
        hm[3, n:] = 0
        kv_lens = []
        for i, st in enumerate(reqs):
            pos = st.seq_len
            blocks = self.kv.blocks_of(st.request_id)
            hm[0, i] = pos + st.rope_delta
            hm[1, i] = blocks[pos // self.bs] * self.bs + pos % self.bs
            hm[2, i] = pos + 1
            hm[3, i] = st.slot_idx
            if device_tokens is None:
                hi[i] = st.last_token()
            kv_lens.append(pos + 1)
        if device_tokens is None:
            hi[n:] = 0
            d["ids"].copy_(d["h_ids"], non_blocking=True)
        else:
            d["ids"][:n].copy_(device_tokens[:n], non_blocking=True)
        d["meta"].copy_(d["h_meta"], non_blocking=True)
        self.kv.flush()
        torch.index_select(self.kv.block_tables, 0, d["meta"][3].long(), out=d["block_tables"])
        return ForwardBatch(
            input_ids=d["ids"], positions=d["meta"][0], slot_mapping=d["meta"][1],
            block_tables=d["block_tables"], seq_lens=d["meta"][2], cu_q=None, logits_indices=None,
            num_seqs=bucket, num_tokens=bucket, max_q_len=1, max_kv_len=max(kv_lens) if kv_lens else 1,
            is_decode=True, config=self.cfg, request_ids=[st.request_id for st in reqs],
            seq_lens_cpu=kv_lens, q_lens_cpu=[1] * n, extras={"num_real": n, "bucket": bucket, "slot_ids": d["meta"][3]})
