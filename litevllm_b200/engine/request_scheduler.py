"""Request bookkeeping: FIFO wait queue, running set with slot indices, per-request output streams.

Thread model: the engine thread mutates scheduling state under the engine lock; HTTP handlers read
streams from an asyncio loop.  Outputs cross threads with ``loop.call_soon_threadsafe``.
Invariants (reference: vllm/engine/request_scheduler.py:12-284 and
docs/design/runtime-hardening-and-serving-correctness.md:68-83): one live id <-> one state, slot and
stream; every stream receives exactly one terminal item (a finished output or an exception);
the terminal item is published before resources are released.
"""
from __future__ import annotations

import asyncio
import time
from collections import deque
from typing import Any

from .errors import InvalidRequestError, RequestRejectedError
from .request_state import RequestState

_DONE = object()


class RequestScheduler:
    def __init__(self, max_active: int, queue_timeout_s: float = 30.0, queue_capacity: int | None = None):
        self.max_active = max_active
        self.queue_timeout_s = queue_timeout_s
        self.queue_capacity = queue_capacity if queue_capacity is not None else 4 * max_active
        self.requests: dict[str, RequestState] = {}
        self.queued: deque[str] = deque()
        self.running: list[str] = []
        self._running_set: set[str] = set()
        self.free_slots: deque[int] = deque(range(max_active))
        self._streams: dict[str, asyncio.Queue] = {}
        # streams of requests that were released before their consumer read (or started to read) them: a short
        # request can finish, or a fatal error can end it, between admission and the consumer's first await
        self._late_streams: dict[str, asyncio.Queue] = {}
        self._stream_loops: dict[str, asyncio.AbstractEventLoop] = {}
        self._sync_outputs: dict[str, list] = {}
        self._terminal_sent: set[str] = set()

    # ------------------------------------------------------------------ admission side
    def enqueue_request(self, state: RequestState, loop: asyncio.AbstractEventLoop | None = None) -> None:
        rid = state.request_id
        if rid in self.requests:
            raise InvalidRequestError(f"duplicate request id {rid!r}")
        if len(self.queued) >= self.queue_capacity:
            raise RequestRejectedError(f"queue full ({self.queue_capacity} waiting requests)", "queue_full")
        self.requests[rid] = state
        self.queued.append(rid)
        if loop is not None:
            self._streams[rid] = asyncio.Queue()
            self._stream_loops[rid] = loop
        else:
            self._sync_outputs[rid] = []

    def expire_queued(self, now: float | None = None) -> list[RequestState]:
        now = time.monotonic() if now is None else now
        expired = []
        while self.queued:
            st = self.requests[self.queued[0]]
            if now - st.arrival_time < self.queue_timeout_s:
                break
            self.queued.popleft()
            expired.append(st)
        return expired

    def admit(self, request_id: str) -> RequestState:
        if not self.free_slots:
            raise RuntimeError("no free slot")
        st = self.requests[request_id]
        try:
            self.queued.remove(request_id)
        except ValueError:
            pass
        st.slot_idx = self.free_slots.popleft()
        st.admitted_time = time.monotonic()
        self.running.append(request_id)
        self._running_set.add(request_id)
        return st

    # ------------------------------------------------------------------ queries
    def get(self, request_id: str) -> RequestState | None:
        return self.requests.get(request_id)

    def is_running(self, request_id: str) -> bool:
        return request_id in self._running_set

    def has_unfinished(self) -> bool:
        return bool(self.queued or self.running)

    def classify_requests(self) -> tuple[list[RequestState], list[RequestState]]:
        """(prefill, decode) in admission order."""
        pre, dec = [], []
        for rid in self.running:
            st = self.requests[rid]
            (pre if st.is_prefill else dec).append(st)
        return pre, dec

    def gauges(self) -> dict[str, int]:
        pre, dec = self.classify_requests()
        return {"queued": len(self.queued), "running": len(self.running), "prefill": len(pre),
                "decode": len(dec), "free_slots": len(self.free_slots), "max_active": self.max_active,
                "queue_capacity": self.queue_capacity}

    # ------------------------------------------------------------------ output side
    def publish_output(self, request_id: str, item: Any) -> None:
        """item: RequestOutput or an Exception (terminal)."""
        terminal = isinstance(item, BaseException) or getattr(item, "finished", False)
        if request_id in self._terminal_sent:
            return
        if terminal:
            self._terminal_sent.add(request_id)
        q = self._streams.get(request_id)
        if q is not None:
            loop = self._stream_loops[request_id]
            try:
                loop.call_soon_threadsafe(q.put_nowait, item)
                if terminal:
                    loop.call_soon_threadsafe(q.put_nowait, _DONE)
            except RuntimeError:
                pass  # loop closed: the consumer is gone
        else:
            box = self._sync_outputs.get(request_id)
            if box is not None:
                box.append(item)

    async def get_request_stream(self, request_id: str):
        q = self._streams.get(request_id) or self._late_streams.get(request_id)
        if q is None:
            raise KeyError(f"no stream for request {request_id!r}")
        try:
            while True:
                item = await q.get()
                if item is _DONE:
                    return
                if isinstance(item, BaseException):
                    raise item
                yield item
        finally:
            self._late_streams.pop(request_id, None)

    def pop_sync_outputs(self, request_id: str) -> list:
        return self._sync_outputs.pop(request_id, [])

    def peek_sync_outputs(self, request_id: str) -> list:
        return self._sync_outputs.get(request_id, [])

    # ------------------------------------------------------------------ teardown
    def release(self, request_id: str) -> RequestState | None:
        """Idempotent removal from every index; returns the state on first call."""
        st = self.requests.pop(request_id, None)
        if st is None:
            return None
        try:
            self.queued.remove(request_id)
        except ValueError:
            pass
        if request_id in self._running_set:
            self._running_set.remove(request_id)
            self.running.remove(request_id)
        if st.slot_idx >= 0:
            self.free_slots.append(st.slot_idx)
            st.slot_idx = -1
        q = self._streams.pop(request_id, None)
        if q is not None:
            self._late_streams[request_id] = q
            while len(self._late_streams) > 1024:        # consumers that never came: drop the oldest
                self._late_streams.pop(next(iter(self._late_streams)))
        self._stream_loops.pop(request_id, None)
        self._terminal_sent.discard(request_id)
        return st

    def all_request_ids(self) -> list[str]:
        return list(self.requests.keys())
