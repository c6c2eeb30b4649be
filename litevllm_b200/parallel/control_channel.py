"""Control channel between rank 0 (which owns the HTTP front end) and the worker ranks.

Offline generation needs no channel: every rank runs the same deterministic engine on the same
prompts.  A server only receives requests on rank 0, so before each step rank 0 publishes a compact
message (new requests, aborts, shutdown) and every worker applies it to its own engine; the engines
then take identical steps.  Transport: the process group's TCP store (host side, independent of
the GPU collectives), with sequence numbers so a lost or reordered message is detected.
A worker that does not see the next message within ``timeout_s`` raises ``RankFailureError``.
"""
from __future__ import annotations

import pickle
import time
from dataclasses import dataclass, field

from ..engine.errors import RankFailureError


@dataclass
class ControlMessage:
    seq: int
    new_requests: list = field(default_factory=list)     # (request_id, prompt token ids, sampling params dict)
    aborts: list = field(default_factory=list)
    shutdown: bool = False
    step: bool = True

    def encode(self) -> bytes:
        return pickle.dumps(self, protocol=pickle.HIGHEST_PROTOCOL)

    @staticmethod
    def decode(data: bytes) -> "ControlMessage":
        msg = pickle.loads(data)
        if not isinstance(msg, ControlMessage):
            raise RankFailureError("malformed control message")
        return msg


class ControlChannel:
    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0, prefix: str = "fi/ctl"):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s = timeout_s
        self.prefix = prefix
        self.seq = 0

    def publish(self, msg: ControlMessage) -> None:
        assert self.rank == 0, "only rank 0 publishes"
        msg.seq = self.seq
        self.store.set(f"{self.prefix}/{self.seq}", msg.encode())
        self.seq += 1

    def receive(self) -> ControlMessage:
        """Blocking receive of the next message in sequence (workers)."""
        key = f"{self.prefix}/{self.seq}"
        deadline = time.monotonic() + self.timeout_s
        while True:
            try:
                if self.store.check([key]):
                    break
            except Exception as e:
                raise RankFailureError(f"control store unreachable: {e!r}") from e
            if time.monotonic() > deadline:
                raise RankFailureError(f"rank {self.rank}: no control message {self.seq} within {self.timeout_s:.1f}s")
            time.sleep(0.0005)
        try:
            msg = ControlMessage.decode(self.store.get(key))
        except RankFailureError:
            raise
        except Exception as e:
            raise RankFailureError(f"rank {self.rank}: cannot decode control message {self.seq}: {e!r}") from e
        if msg.seq != self.seq:
            raise RankFailureError(f"rank {self.rank}: expected control message {self.seq}, got {msg.seq}")
        self.seq += 1
        return msg

    def apply(self, engine, msg: ControlMessage) -> bool:
        """Apply a message to a worker engine; returns False when the worker should stop."""
        from ..sampling_params import SamplingParams
        for rid in msg.aborts:
            engine.abort_request(rid)
        for rid, ids, sp in msg.new_requests:
            engine.add_request(rid, {"prompt_token_ids": ids}, SamplingParams(**sp))
        return not msg.shutdown
