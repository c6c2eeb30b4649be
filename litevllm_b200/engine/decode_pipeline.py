"""Pipelined decode: step k+1 is launched before the host has looked at the tokens of step k.

While the set of decoding requests is unchanged, one step costs the host only
  * a vectorised (numpy) update of positions / slots / sequence lengths in a pinned ring slot and
    ONE asynchronous H2D copy of that metadata,
  * a device-to-device copy of the previous step's sampled tokens into the input buffer,
  * a CUDA-graph replay (model forward + arg-max),
  * an asynchronous D2H copy of the sampled tokens into a pinned ring slot plus an event,
after which the host processes the tokens of the *previous* step (stop checks, streaming) while the
GPU runs the current one.  A request that stops early (EOS / stop string) is noticed one step late;
the extra token the GPU computed for it is dropped.  Any change of the request set drains the
pipeline and the next step starts it again.  Only greedy, unconstrained, penalty-free requests
qualify; everything else takes the synchronous path of :class:`DecodeExecutor`.
The reference builds and syncs every step (vllm/engine/decode_executor.py:29-70,
vllm/engine/sampling/sampler.py:18-40: one ``.item()`` per row per step).
"""
from __future__ import annotations

import numpy as np
import torch

from .request_state import RequestState

RING = 4


class DecodePipeline:
    def __init__(self, executor, builder, kv_manager):
        self.ex = executor
        self.builder = builder
        self.kv = kv_manager
        self.device = builder.device
        self.active = False
        self.key: tuple = ()
        self.reqs: list[RequestState] = []
        self.inflight: list[tuple] = []     # (event, pinned token slot index, n real rows)
        self.step_idx = 0
        self.launched_steps = 0
        self._bufs: dict[int, dict] = {}

    # ------------------------------------------------------------------ eligibility
    @staticmethod
    def eligible(st: RequestState) -> bool:
        sp = st.sampling_params
        return (sp.is_greedy and not sp.has_penalties and not sp.logit_bias
                and st.structured_output_constraint is None and st.lora_request is None)

    def _buffers(self, bucket: int) -> dict:
        b = self._bufs.get(bucket)
        if b is None:
            pin = self.device.type == "cuda"
            b = {"h_meta": torch.zeros(RING, 4, bucket, dtype=torch.int32, pin_memory=pin),
                 "h_tok": torch.zeros(RING, bucket, dtype=torch.int64, pin_memory=pin),
                 "next_ids": torch.zeros(bucket, dtype=torch.int64, device=self.device)}
            self._bufs[bucket] = b
        return b

    # ------------------------------------------------------------------ lifecycle
    @torch.inference_mode()
    def start(self, reqs: list[RequestState]) -> None:
        """Begin pipelining for this request set; the first step takes its input ids from the host."""
        self.reqs = list(reqs)
        self.key = tuple(st.request_id for st in reqs)
        n = len(reqs)
        self.n = n
        self.bucket = self.builder.bucket_for(n)
        self.dec = self.builder._decode_buffers(self.bucket)
        self.buf = self._buffers(self.bucket)
        bs = self.kv.block_size
        self.pos = np.array([st.seq_len for st in reqs], dtype=np.int64)
        self.slot_ids = np.array([st.slot_idx for st in reqs], dtype=np.int32)
        self.rope_delta = np.array([st.rope_delta for st in reqs], dtype=np.int64)
        self.limit = np.array([st.sampling_params.max_tokens - len(st.generated_ids) for st in reqs], dtype=np.int64)
        self.bs = bs
        self.launched_steps = 0
        self.step_idx = 0
        self.inflight = []
        self.active = True
        hi = self.dec["h_ids"].numpy()
        hi[:n] = [st.last_token() for st in reqs]
        hi[n:] = 0
        self.dec["ids"].copy_(self.dec["h_ids"], non_blocking=True)
        self._first = True

    def can_launch(self) -> bool:
        """False once some request has had all of its remaining tokens launched."""
        return bool((self.limit - self.launched_steps > 0).all())

    @torch.inference_mode()
    def launch(self, read_back: bool = True) -> None:
        n, bucket = self.n, self.bucket
        ring = self.step_idx % RING
        # blocks for the token written by this step
        pos = self.pos
        new_block = (pos % self.bs) == 0
        if self._first or new_block.any():
            for i in np.nonzero(new_block | self._first)[0]:
                self.kv.ensure_blocks(self.reqs[i].request_id, int(pos[i]) + 1)
            self.blk_rows = [self.kv.blocks_of(st.request_id) for st in self.reqs]
        blk = np.fromiter((self.blk_rows[i][int(pos[i]) // self.bs] for i in range(n)), dtype=np.int64, count=n)
        hm = self.buf["h_meta"][ring].numpy()
        hm[0, :n] = pos + self.rope_delta
        hm[1, :n] = blk * self.bs + pos % self.bs
        hm[2, :n] = pos + 1
        hm[3, :n] = self.slot_ids
        hm[0, n:] = 0
        hm[1, n:] = -1
        hm[2, n:] = 0
        hm[3, n:] = 0
        d = self.dec
        d["meta"].copy_(self.buf["h_meta"][ring], non_blocking=True)
        self._first = False
        self.kv.flush()
        # the captured step gathers the block tables, runs the model and leaves the greedy tokens in
        # d["ids"], which is also where the next step reads its input ids
        self.ex.replay_or_capture(self.bucket, self.reqs, int(pos.max()) + 1)
        if read_back:
            self.buf["h_tok"][ring].copy_(d["ids"], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self.inflight.append((ev, ring, n))
        else:
            self.inflight.append((None, ring, n))
        self.pos = pos + 1
        for st in self.reqs:
            st.seq_len += 1
        self.launched_steps += 1
        self.step_idx += 1

    @torch.inference_mode()
    def collect_oldest(self) -> list[int] | None:
        """Wait for the oldest in-flight step and return its tokens (one per request)."""
        if not self.inflight:
            return None
        ev, ring, n = self.inflight.pop(0)
        if ev is None:
            torch.cuda.current_stream().synchronize()
            self.buf["h_tok"][ring].copy_(self.dec["ids"])
        else:
            ev.synchronize()
        return self.buf["h_tok"][ring][:n].tolist()

    def stop(self) -> None:
        self.active = False
        self.inflight = []
        self.reqs = []
        self.key = ()
