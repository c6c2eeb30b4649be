"""Failure detection for multi-rank serving, all on the host.

* ``Heartbeat``: every rank bumps a counter in the TCP store from a daemon thread; ``check`` reports
  ranks whose counter has not moved for ``timeout_s``.  The engine calls ``raise_if_dead`` between
  steps, so a missing peer is noticed before the next collective is launched.
* ``decode_status``: maps the device status word that the bounded waits of the fused kernels set
  (csrc/common/ptx.cuh) to an exception; the context stays usable after a time-out.
No device fault is ever provoked: a rank "fails" by stopping its heartbeat, raising, or exiting
between steps.  The reference has no multi-rank runtime; its single-process failure handling
(fatal background error -> all streams fail, vllm/engine/lite_engine.py:873-892) is kept as is.
"""
from __future__ import annotations

import threading
import time

from ..engine.errors import ExecutionStepError, RankFailureError

STATUS_NAMES = {0: "ok", 1: "timeout waiting for data", 2: "timeout waiting for a free pipeline slot",
                3: "timeout waiting for the accumulator", 4: "timeout waiting for a peer rank",
                5: "bad argument"}


def decode_status(code: int) -> None:
    if code == 0:
        return
    name = STATUS_NAMES.get(code, f"unknown status {code}")
    if code == 4:
        raise RankFailureError(f"a fused collective kernel gave up: {name}")
    raise ExecutionStepError(f"a device kernel reported: {name}")


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval_s: float = 0.5, timeout_s: float = 10.0,
                 prefix: str = "fi/hb", clock=time.monotonic):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s, self.prefix = interval_s, timeout_s, prefix
        self.clock = clock
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._last_seen: dict[int, tuple[int, float]] = {}
        self.beats = 0

    def beat_once(self) -> None:
        self.beats += 1
        self.store.set(f"{self.prefix}/{self.rank}", str(self.beats).encode())

    def start(self) -> None:
        if self._thread is not None:
            return
        self.beat_once()

        def loop():
            while not self._stop.wait(self.interval_s):
                try:
                    self.beat_once()
                except Exception:
                    return
        self._thread = threading.Thread(target=loop, name="fi-heartbeat", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval_s + 1)
            self._thread = None

    def check(self) -> list[int]:
        """Ranks considered dead: never seen, or counter unchanged for longer than ``timeout_s``."""
        now = self.clock()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            key = f"{self.prefix}/{r}"
            try:
                val = int(self.store.get(key).decode()) if self.store.check([key]) else -1
            except Exception:
                val = -1
            prev = self._last_seen.get(r)
            if prev is None or val != prev[0]:
                self._last_seen[r] = (val, now)
                if prev is None and val < 0:
                    self._last_seen[r] = (-1, now)
                continue
            if now - prev[1] > self.timeout_s:
                dead.append(r)
        return dead

    def raise_if_dead(self) -> None:
        dead = self.check()
        if dead:
            raise RankFailureError(f"rank(s) {dead} stopped sending heartbeats for more than {self.timeout_s:.1f}s")
