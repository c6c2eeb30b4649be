"""Serving on several ranks: rank 0 owns the HTTP front end, every rank runs the same engine.

The engines must take identical steps on identical request sets (tensor/expert parallel kernels
exchange partial results inside every step).  Requests only arrive at rank 0, so rank 0's stepping
loop publishes, BEFORE every step, one control message with the requests admitted and the aborts
issued since the previous step plus the decision whether a step follows; workers apply the message
to their engine and take the step.  A request is sent as token ids + resolved sampling parameters
(after rank 0's validation, caps and tokenisation), with an explicit seed for sampled requests, so
that every rank builds the same request state.  While idle, rank 0 sends keep-alive messages so a
worker can tell a quiet server from a dead rank 0; a worker that misses messages for ``timeout_s``
raises ``RankFailureError``; a dead worker is noticed by rank 0 through the heartbeat hook of
``DistributedHandle`` and fails the engine, which turns ``/readyz`` to 503.
The reference serves from a single process (vllm/entrypoints/openai/api_server.py:385-434,
vllm/engine/async_driver.py:64-125); this is the multi-GPU extension of that contract.
"""
from __future__ import annotations

import dataclasses
import secrets

from ..engine.errors import InvalidRequestError
from .control_channel import ControlChannel, ControlMessage


def sampling_params_to_wire(sp) -> dict:
    d = dataclasses.asdict(sp)
    return d


class ServingCoordinator:
    """Rank 0 side.  All methods are called with the engine lock held."""

    def __init__(self, channel: ControlChannel):
        self.channel = channel
        self._new: list = []
        self._aborts: list = []
        self.messages = 0
        self.closed = False

    @staticmethod
    def prepare_params(sampling_params):
        """Give a sampled request an explicit seed so that every rank draws the same tokens."""
        if sampling_params is not None and not sampling_params.is_greedy and sampling_params.seed is None:
            sampling_params = sampling_params.clone()
            sampling_params.seed = secrets.randbits(62)
        return sampling_params

    @staticmethod
    def check_supported(lora_request, multi_modal_data) -> None:
        if lora_request is not None or multi_modal_data:
            raise InvalidRequestError("LoRA adapters and image inputs are not forwarded to worker ranks; "
                                      "serve them from a single-GPU engine")

    def record_request(self, st) -> None:
        self._new.append((st.request_id, list(st.prompt_token_ids), sampling_params_to_wire(st.sampling_params)))

    def record_abort(self, request_id: str) -> None:
        self._aborts.append(request_id)

    def before_step(self, engine) -> bool:
        """Publish what changed and whether a step follows; returns that decision."""
        step = engine.has_unfinished_requests()
        if not (step or self._new or self._aborts):
            return False
        self.channel.publish(ControlMessage(seq=0, new_requests=self._new, aborts=self._aborts, step=step))
        self._new, self._aborts = [], []
        self.messages += 1
        return step

    def keepalive(self) -> None:
        if not self.closed:
            self.channel.publish(ControlMessage(seq=0, step=False))
            self.messages += 1

    def shutdown(self) -> None:
        if not self.closed:
            self.closed = True
            self.channel.publish(ControlMessage(seq=0, step=False, shutdown=True))


def worker_serve_loop(engine, channel: ControlChannel, on_step=None) -> int:
    """Worker ranks: apply rank 0's messages and step in lockstep until told to shut down.  Returns the
    number of steps taken.  ``on_step(outputs)`` (optional) sees what every step produced."""
    steps = 0
    while True:
        msg = channel.receive()
        alive = channel.apply(engine, msg)
        if msg.step:
            outs = engine.step()
            steps += 1
            if on_step is not None:
                on_step(outs)
        if not alive:
            return steps


def make_channel(state, timeout_s: float = 60.0) -> ControlChannel:
    import torch.distributed as dist
    store = dist.distributed_c10d._get_default_store()
    return ControlChannel(store, state.rank, state.world_size, timeout_s=timeout_s)
