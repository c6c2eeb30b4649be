"""Multi-rank serving on 2 GPUs: rank 0 answers HTTP requests through FastAPI's TestClient with a
tensor-parallel engine whose collectives are the fused in-kernel ones; rank 1 mirrors the admitted
requests through the control channel and runs every step with it.  Both ranks must have produced the same
tokens.  Child processes, one per GPU; NVLS off for NCCL, plain peer stores in the fused kernels."""
import json
import os
import tempfile

import pytest

from litevllm_b200.parallel.launcher import spawn

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _serve_worker(rank, world, out_dir):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from litevllm_b200.entrypoints.openai import api_server as srv
    eng = srv.build_engine("synthetic:tiny-llama-test", dtype="bfloat16", max_num_seqs=4, max_model_len=128,
                           tensor_parallel_size=world, comm_backend="fused")
    produced: dict = {}

    def on_step(outs):
        for o in outs:
            if o is not None and o.finished:
                produced[o.request_id] = list(o.outputs[0].token_ids)

    if eng.is_worker_rank:
        steps = eng.serve_as_worker(on_step)
        with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
            json.dump({"tokens": sorted(produced.values()), "steps": steps}, f)
        eng.shutdown()
        return
    from fastapi.testclient import TestClient
    orig_step = eng.engine.step

    def recording_step():
        outs = orig_step()
        on_step(outs)
        return outs
    eng.engine.step = recording_step
    srv.engine, srv.served_model = eng, "tiny"
    client = TestClient(srv.app)
    assert client.get("/readyz").status_code == 200
    body = {"model": "tiny", "messages": [{"role": "user", "content": "hello there"}], "max_tokens": 6, "temperature": 0}
    r = client.post("/v1/chat/completions", json=body)
    assert r.status_code == 200 and r.json()["usage"]["completion_tokens"] == 6
    r2 = client.post("/v1/chat/completions", json=dict(body, temperature=0.8, top_p=0.9, max_tokens=5,
                                                       messages=[{"role": "user", "content": "second"}]))
    assert r2.status_code == 200
    with client.stream("POST", "/v1/chat/completions", json=dict(body, stream=True, max_tokens=4)) as s:
        lines = [ln for ln in s.iter_lines() if ln.startswith("data:")]
    assert lines[-1] == "data: [DONE]"
    from litevllm_b200.parallel import state as pstate
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump({"tokens": sorted(produced.values()), "backend": pstate.get_state().comm_backend,
                   "self_test": pstate.get_state().self_test}, f)
    eng.shutdown()


def test_two_gpu_server_with_fused_collectives():
    with tempfile.TemporaryDirectory() as d:
        spawn(_serve_worker, 2, args=(d,), port=29581)
        r0 = json.load(open(os.path.join(d, "rank0.json")))
        r1 = json.load(open(os.path.join(d, "rank1.json")))
    assert r0["backend"] == "fused" and r0["self_test"]["allreduce_one_hop"]
    assert len(r0["tokens"]) == 3 and r0["tokens"] == r1["tokens"]
