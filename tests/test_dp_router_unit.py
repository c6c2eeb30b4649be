"""The data-parallel router against an in-memory store: request forwarding, stream delivery when the replica
finishes before the consumer starts to read, abort, in-flight accounting."""
import asyncio
import pickle
import threading
import time

from litevllm_b200.outputs import CompletionOutput, RequestOutput
from litevllm_b200.parallel.dp_serving import DataParallelRouter, ReplicaLink


class FakeStore:
    def __init__(self):
        self.d, self.lock = {}, threading.Lock()

    def set(self, k, v):
        with self.lock:
            self.d[k] = v

    def get(self, k):
        with self.lock:
            return self.d[k]

    def check(self, keys):
        with self.lock:
            return all(k in self.d for k in keys)

    def delete_key(self, k):
        with self.lock:
            return self.d.pop(k, None) is not None


def _out(rid, toks, finished):
    comp = CompletionOutput(index=0, token_ids=list(toks), text="x" * len(toks), decode=None, cumulative_logprob=0.0,
                            finish_reason="length" if finished else None)
    return RequestOutput(request_id=rid, prompt=None, prompt_token_ids=[1, 2], outputs=[comp], finished=finished,
                         finish_reason="length" if finished else None, metrics={})


def test_router_delivers_to_a_late_consumer_and_keeps_count():
    store = FakeStore()
    router = DataParallelRouter(store, replicas=2)
    replica = ReplicaLink(store, 1)                 # the replica's end of the same mailboxes
    loop = asyncio.new_event_loop()
    try:
        assert router.choose() == 0
        router.note_local("local-1")
        assert router.choose() == 1                  # rank 0 is busier now
        router.submit_remote(1, "r1", [5, 6, 7], {"max_tokens": 2}, loop)
        msg = replica.poll_down()
        assert msg[0] == "req" and msg[1] == "r1" and msg[2] == [5, 6, 7]
        assert router.stats()["inflight"] == [1, 1] and router.is_remote("r1")
        # the replica finishes the whole request before anybody reads the stream
        replica.send_up(("out", _out("r1", [9], False)))
        replica.send_up(("out", _out("r1", [9, 4], True)))
        for _ in range(400):
            if router.stats()["inflight"][1] == 0:
                break
            time.sleep(0.005)
        assert router.stats()["inflight"] == [1, 0]
        assert router.is_remote("r1")                # still known: its consumer has not come yet

        async def drain(rid):
            return [o async for o in router.stream(rid)]

        outs = loop.run_until_complete(asyncio.wait_for(drain("r1"), 5))
        assert [o.finished for o in outs] == [False, True] and outs[-1].outputs[0].token_ids == [9, 4]
        assert not router.is_remote("r1")            # consumed: forgotten
        # abort of a remote request: the replica is told, the stream ends with an error, the count drops once
        router.submit_remote(1, "r2", [1], {"max_tokens": 50}, loop)
        assert replica.poll_down()[1] == "r2"
        assert router.abort("r2") and replica.poll_down() == ("abort", "r2")
        replica.send_up(("out", _out("r2", [3], True)))          # a late final output must not be counted twice
        time.sleep(0.05)
        assert router.stats()["inflight"] == [1, 0]
        try:
            loop.run_until_complete(asyncio.wait_for(drain("r2"), 5))
            raised = False
        except RuntimeError as e:
            raised = "aborted" in str(e)
        assert raised
        router.finish_local("local-1")
        assert router.stats()["inflight"] == [0, 0] and not router.abort("unknown")
    finally:
        router._stop.set()
        router._pump.join(timeout=2)
        loop.close()
