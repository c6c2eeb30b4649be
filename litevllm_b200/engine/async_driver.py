"""Background stepping loop: one daemon worker thread calls ``engine.step()`` under the engine lock
while work exists, sleeps ``min_step_interval_s`` between steps and idles on a wake-up queue.
Any exception in a step is wrapped as ``BackgroundLoopError``, handed to
``engine.handle_background_error`` (which fails every stream) and stops the loop.
Reference: vllm/engine/async_driver.py:18-125."""
from __future__ import annotations

import queue
import threading
import time

from .errors import BackgroundLoopError


class AsyncDriver:
    def __init__(self, engine, lock: threading.RLock, min_step_interval_s: float = 0.001,
                 idle_timeout_s: float = 1.0, sleep_fn=time.sleep, coordinator=None):
        # coordinator (multi-rank serving, rank 0 only): told before every step which requests were admitted or
        # aborted since the last one, so that the worker ranks can mirror this engine step by step
        self.coordinator = coordinator
        self.engine = engine
        self.lock = lock
        self.min_step_interval_s = min_step_interval_s
        self.idle_timeout_s = idle_timeout_s
        self._sleep = sleep_fn
        self._wake: queue.Queue = queue.Queue()
        self._thread: threading.Thread | None = None
        self._running = False
        self._start_lock = threading.Lock()
        self.steps = 0
        self.idle_wakeups = 0
        self.errors = 0
        self.last_error: BaseException | None = None

    def start(self) -> None:
        with self._start_lock:
            if self._thread is not None and self._thread.is_alive():
                return
            self._running = True
            self._thread = threading.Thread(target=self._run_loop, name="fi-async-driver", daemon=True)
            self._thread.start()

    def notify_new_work(self) -> None:
        self.start()
        self._wake.put(1)

    def _run_loop(self) -> None:
        while self._running:
            try:
                with self.lock:
                    if self.coordinator is not None:
                        busy = self.coordinator.before_step(self.engine)
                    else:
                        busy = self.engine.has_unfinished_requests()
                    if busy:
                        self.engine.step()
                        self.steps += 1
            except BaseException as e:  # noqa: BLE001 - the loop must never die silently
                self.errors += 1
                err = e if isinstance(e, BackgroundLoopError) else BackgroundLoopError(f"engine step failed: {e!r}")
                err.__cause__ = e
                self.last_error = err
                try:
                    self.engine.handle_background_error(err)
                finally:
                    self._running = False
                return
            if busy:
                if self.min_step_interval_s > 0:
                    self._sleep(self.min_step_interval_s)
            else:
                try:
                    self._wake.get(timeout=self.idle_timeout_s)
                    self.idle_wakeups += 1
                except queue.Empty:
                    if self.coordinator is not None:      # a quiet server still tells its workers that it is alive
                        with self.lock:
                            self.coordinator.keepalive()
                # drain extra wake tokens
                while True:
                    try:
                        self._wake.get_nowait()
                    except queue.Empty:
                        break

    @property
    def is_running(self) -> bool:
        return self._running and self._thread is not None and self._thread.is_alive()

    def shutdown(self, timeout: float = 5.0) -> None:
        if self.coordinator is not None:
            with self.lock:
                self.coordinator.shutdown()
        self._running = False
        self._wake.put(0)
        t = self._thread
        if t is not None and t.is_alive() and t is not threading.current_thread():
            t.join(timeout)

    def stats(self) -> dict:
        return {"running": self.is_running, "steps": self.steps, "idle_wakeups": self.idle_wakeups,
                "errors": self.errors, "last_error": repr(self.last_error) if self.last_error else None}
