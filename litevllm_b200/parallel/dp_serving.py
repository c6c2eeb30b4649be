"""Serving with data-parallel replicas: rank 0 owns the HTTP front end and one engine, every other rank
runs a whole engine of its own, and each request is served by exactly one replica.

Rank 0 validates and tokenises a request with its own request builder, picks the replica with the fewest
requests in flight (itself included) and, for a remote replica, sends the request down that replica's
mailbox; the replica adds it to its engine, steps, and sends every ``RequestOutput`` back up.  A pump
thread on rank 0 feeds those outputs into the per-request stream the HTTP handler is reading, so a caller
cannot tell where its request ran.  Mailboxes are two numbered key sequences per replica in the process
group's TCP store (host side, no GPU collective involved), consumed keys are deleted.

Replicas are independent: they do not step in lockstep and share no GPU state, so a slow request on one
does not hold up the others.  The reference serves from one process and one GPU
(vllm/entrypoints/openai/api_server.py:385-434); this is the scale-out counterpart of the single-engine
server, next to the lockstep tensor-parallel form in parallel/serving.py.
"""
from __future__ import annotations

import asyncio
import pickle
import threading
import time

from ..engine.errors import EngineFatalError, RankFailureError


class ReplicaLink:
    """Both directions between rank 0 and one replica.  ``down``: rank 0 -> replica, ``up``: replica -> rank 0."""

    def __init__(self, store, replica: int, prefix: str = "fi/dp"):
        self.store, self.replica = store, replica
        self.prefix = f"{prefix}/{replica}"
        self._sent = {"down": 0, "up": 0}
        self._seen = {"down": 0, "up": 0}
        self._lock = threading.Lock()

    def _send(self, way: str, obj) -> None:
        with self._lock:
            seq = self._sent[way]
            self._sent[way] += 1
        self.store.set(f"{self.prefix}/{way}/{seq}", pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL))

    def _poll(self, way: str):
        key = f"{self.prefix}/{way}/{self._seen[way]}"
        try:
            if not self.store.check([key]):
                return None
            data = self.store.get(key)
            self.store.delete_key(key)
        except Exception as e:
            raise RankFailureError(f"replica {self.replica}: mailbox store unreachable: {e!r}") from e
        self._seen[way] += 1
        return pickle.loads(data)

    def send_down(self, obj) -> None: self._send("down", obj)
    def send_up(self, obj) -> None: self._send("up", obj)
    def poll_down(self): return self._poll("down")
    def poll_up(self): return self._poll("up")


def replica_serve_loop(engine, link: ReplicaLink, idle_sleep_s: float = 0.001, on_step=None) -> int:
    """Ranks other than 0: take requests from the mailbox, step the local engine while it has work and send
    every output up.  Returns the number of steps taken when rank 0 says shutdown."""
    from ..sampling_params import SamplingParams
    steps = 0
    while True:
        while True:
            msg = link.poll_down()
            if msg is None:
                break
            kind = msg[0]
            if kind == "shutdown":
                try:
                    link.send_up(("bye",))      # rank 0 keeps the store up until every replica has read its shutdown
                except Exception:
                    pass
                return steps
            if kind == "abort":
                engine.abort_request(msg[1])
            elif kind == "req":
                _, rid, ids, sp = msg
                try:
                    engine.add_request(rid, {"prompt_token_ids": ids}, SamplingParams(**sp))
                except Exception as e:     # rejected here (e.g. no capacity): the caller's stream gets the error
                    link.send_up(("error", rid, f"{type(e).__name__}: {e}"))
        if engine.has_unfinished_requests():
            outs = engine.step()
            steps += 1
            for o in outs:
                if o is not None:
                    link.send_up(("out", o))
            if on_step is not None:
                on_step(outs)
        else:
            time.sleep(idle_sleep_s)


class DataParallelRouter:
    """Rank 0: replica choice, request forwarding and the pump that turns mailbox traffic into streams."""

    def __init__(self, store, replicas: int, poll_sleep_s: float = 0.0005):
        self.replicas = replicas
        self.links = {r: ReplicaLink(store, r) for r in range(1, replicas)}
        self.inflight = [0] * replicas
        self.owner: dict[str, int] = {}
        self._streams: dict[str, tuple[asyncio.Queue, asyncio.AbstractEventLoop]] = {}
        self._done: dict[str, None] = {}        # finished remotely, stream not read to its end yet (oldest first)
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._poll_sleep_s = poll_sleep_s
        self.error: BaseException | None = None
        self._pump = threading.Thread(target=self._pump_loop, name="fi-dp-pump", daemon=True)
        self._pump.start()

    # ---------------------------------------------------------------- routing
    def choose(self) -> int:
        with self._lock:
            return min(range(self.replicas), key=lambda r: (self.inflight[r], r))

    def note_local(self, request_id: str) -> None:
        with self._lock:
            self.owner[request_id] = 0
            self.inflight[0] += 1

    def finish_local(self, request_id: str) -> None:
        with self._lock:
            if self.owner.pop(request_id, None) == 0:
                self.inflight[0] = max(0, self.inflight[0] - 1)

    def submit_remote(self, replica: int, request_id: str, prompt_ids: list[int], sampling: dict,
                      loop: asyncio.AbstractEventLoop) -> None:
        if self.error is not None:
            raise EngineFatalError(f"data-parallel pump stopped: {self.error!r}")
        with self._lock:
            self.owner[request_id] = replica
            self.inflight[replica] += 1
            self._streams[request_id] = (asyncio.Queue(), loop)
        self.links[replica].send_down(("req", request_id, list(prompt_ids), sampling))

    def is_remote(self, request_id: str) -> bool:
        return self.owner.get(request_id, 0) != 0

    async def stream(self, request_id: str):
        """Outputs of a remote request.  The queue outlives the request until its consumer has read it: a short
        request can finish on its replica before the consumer awaits the stream for the first time."""
        q, _ = self._streams[request_id]
        try:
            while True:
                item = await q.get()
                if isinstance(item, BaseException):
                    raise item
                yield item
                if getattr(item, "finished", False):
                    return
        finally:
            with self._lock:
                self._streams.pop(request_id, None)
                self.owner.pop(request_id, None)
                self._done.pop(request_id, None)

    def abort(self, request_id: str) -> bool:
        with self._lock:
            r = self.owner.get(request_id, 0)
        if r == 0:
            return False
        self.links[r].send_down(("abort", request_id))
        self._finish_remote(request_id, RuntimeError(f"request {request_id} aborted"))
        return True

    # ---------------------------------------------------------------- pump
    def _deliver(self, request_id: str, item) -> None:
        entry = self._streams.get(request_id)
        if entry is not None:
            q, loop = entry
            loop.call_soon_threadsafe(q.put_nowait, item)

    def _finish_remote(self, request_id: str, terminal=None) -> None:
        """Book-keeping first, delivery second: the consumer may drop the stream the moment it sees the last item."""
        with self._lock:
            r = self.owner.get(request_id)
            if r and request_id not in self._done:
                self.inflight[r] = max(0, self.inflight[r] - 1)
                self._done[request_id] = None
                while len(self._done) > 1024:           # consumers that never came back: forget the oldest
                    old = next(iter(self._done))
                    self._done.pop(old)
                    self.owner.pop(old, None)
                    self._streams.pop(old, None)
        if terminal is not None:
            self._deliver(request_id, terminal)

    def _pump_loop(self) -> None:
        try:
            while not self._stop.is_set():
                busy = False
                for link in self.links.values():
                    msg = link.poll_up()
                    while msg is not None:
                        busy = True
                        if msg[0] == "out":
                            out = msg[1]
                            if out.finished:
                                self._finish_remote(out.request_id, out)
                            else:
                                self._deliver(out.request_id, out)
                        elif msg[0] == "error":
                            from ..engine.errors import RequestRejectedError
                            self._finish_remote(msg[1], RequestRejectedError(msg[2]))
                        msg = link.poll_up()
                if not busy:
                    time.sleep(self._poll_sleep_s)
        except BaseException as e:       # the store went away: fail the open streams instead of hanging them
            self.error = e
            for rid in list(self._streams):
                self._finish_remote(rid, EngineFatalError(f"data-parallel pump stopped: {e!r}"))

    def shutdown(self, wait_s: float = 5.0) -> None:
        """Tell every replica to stop and wait (bounded) for each to acknowledge: rank 0 hosts the mailbox store, so
        leaving before a replica has read its shutdown message would show up there as a lost store."""
        self._stop.set()
        self._pump.join(timeout=2.0)
        waiting = set()
        for r, link in self.links.items():
            try:
                link.send_down(("shutdown",))
                waiting.add(r)
            except Exception:
                pass
        deadline = time.monotonic() + wait_s
        while waiting and time.monotonic() < deadline:
            for r in list(waiting):
                try:
                    msg = self.links[r].poll_up()
                except Exception:
                    waiting.discard(r)
                    continue
                if msg is not None and msg[0] == "bye":
                    waiting.discard(r)
            if waiting:
                time.sleep(0.002)

    def stats(self) -> dict:
        with self._lock:
            return {"replicas": self.replicas, "inflight": list(self.inflight)}
