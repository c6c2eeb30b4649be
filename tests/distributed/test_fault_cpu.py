"""Control channel and failure detection with gloo/CPU ranks and an in-memory store: a rank that
stops its heartbeat, a dropped message, a malformed message, a worker that exits between steps."""
import time

import pytest
import torch.distributed as dist

from litevllm_b200.engine.errors import ExecutionStepError, RankFailureError
from litevllm_b200.parallel.control_channel import ControlChannel, ControlMessage
from litevllm_b200.parallel.fault import Heartbeat, decode_status
from litevllm_b200.parallel.launcher import spawn


class DictStore:
    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v

    def get(self, k):
        return self.d[k]

    def check(self, keys):
        return all(k in self.d for k in keys)


def test_heartbeat_detects_a_silent_rank():
    store = DictStore()
    t = [0.0]
    a = Heartbeat(store, 0, 3, timeout_s=5.0, clock=lambda: t[0])
    b = Heartbeat(store, 1, 3, timeout_s=5.0, clock=lambda: t[0])
    a.beat_once(); b.beat_once()
    assert a.check() == []                 # first observation only records
    t[0] = 3.0
    b.beat_once()
    assert a.check() == []                 # rank 2 silent but still inside the window
    t[0] = 6.0
    b.beat_once()
    assert a.check() == [2]                # rank 2 never beat
    t[0] = 20.0
    assert sorted(a.check()) == [1, 2]     # rank 1 stopped as well
    with pytest.raises(RankFailureError):
        a.raise_if_dead()


def test_control_channel_orders_and_detects_loss():
    store = DictStore()
    tx = ControlChannel(store, 0, 2)
    rx = ControlChannel(store, 1, 2, timeout_s=0.05)
    tx.publish(ControlMessage(0, new_requests=[("r0", [1, 2, 3], {"max_tokens": 4})]))
    tx.publish(ControlMessage(0, aborts=["r0"]))
    m0, m1 = rx.receive(), rx.receive()
    assert (m0.seq, m1.seq) == (0, 1) and m0.new_requests[0][0] == "r0" and m1.aborts == ["r0"]
    with pytest.raises(RankFailureError, match="no control message"):
        rx.receive()                       # nothing published: bounded wait, then an error
    # a dropped message: sequence 2 is lost, 3 arrives -> the receiver still waits for 2 and times out
    tx.seq = 3
    tx.publish(ControlMessage(0))
    with pytest.raises(RankFailureError):
        rx.receive()
    # a malformed payload
    store.set("fi/ctl/2", b"garbage")
    with pytest.raises(RankFailureError, match="decode"):
        rx.receive()


def test_status_word_decoding():
    decode_status(0)
    with pytest.raises(RankFailureError):
        decode_status(4)
    with pytest.raises(ExecutionStepError):
        decode_status(1)


def _worker_exits_between_steps(rank, world):
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, interval_s=0.05, timeout_s=0.5)
    hb.start()
    chan = ControlChannel(store, rank, world, timeout_s=5.0)
    if rank == 0:
        for step in range(3):
            chan.publish(ControlMessage(0))
            time.sleep(0.1)
        # rank 1 leaves after step 1 (between steps, nothing in flight); rank 0 must notice on the host
        deadline = time.time() + 10
        while time.time() < deadline and hb.check() != [1]:
            time.sleep(0.1)
        assert hb.check() == [1], "rank 0 did not notice that rank 1 left"
        with pytest.raises(RankFailureError):
            hb.raise_if_dead()
    else:
        chan.receive()
        chan.receive()
        hb.stop()           # simulate the rank going away between steps
        time.sleep(3.0)
    hb.stop()


def test_rank_leaving_between_steps_is_noticed_on_the_host():
    spawn(_worker_exits_between_steps, 2, port=29561)
