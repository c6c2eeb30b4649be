"""Data parallelism as gloo ranks on the CPU: two replicas of a tiny model share one ``generate`` call;
every rank must return the whole list, in order, equal to what one engine alone produces."""
import json
import os
import tempfile

from litevllm_b200.parallel.launcher import spawn

PROMPTS = [[5, 9, 14, 3], [7, 7, 2], [11, 4, 6, 8, 1], [3], [9, 2, 2, 2, 5, 6], [12, 13]]


def _kwargs():
    return dict(dtype="float32", device="cpu", max_num_seqs=4, max_model_len=64)


def _dp_worker(rank, world, out_dir):
    from litevllm_b200 import LLM, SamplingParams
    llm = LLM("synthetic:tiny-llama-test", data_parallel_size=world, **_kwargs())
    outs = llm.generate([list(p) for p in PROMPTS], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump({"tokens": [list(o.outputs[0].token_ids) for o in outs],
                   "served_here": llm.engine.stats().get("requests_finished", None)}, f)
    llm.shutdown()


def test_two_replicas_return_the_whole_list_in_order():
    from litevllm_b200 import LLM, SamplingParams
    single = LLM("synthetic:tiny-llama-test", **_kwargs())
    want = [list(o.outputs[0].token_ids) for o in
            single.generate([list(p) for p in PROMPTS], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))]
    single.shutdown()
    with tempfile.TemporaryDirectory() as d:
        spawn(_dp_worker, 2, args=(d,), port=29571)
        got = [json.load(open(os.path.join(d, f"rank{r}.json"))) for r in range(2)]
    assert got[0]["tokens"] == want and got[1]["tokens"] == want


def test_replicas_of_sharded_groups_are_offline_only():
    """The parallel layout accepts replicas of tensor-parallel groups; the server does not route to them."""
    import pytest

    from litevllm_b200.config.config_builder import build_vllm_config
    from litevllm_b200.config.parallel_config import ParallelConfig
    from litevllm_b200.engine.async_llm import AsyncLLM
    pc = ParallelConfig.from_env(tp=2, dp=2)
    assert pc.world_size == 2 and pc.data_parallel_size == 2
    cfg = build_vllm_config("synthetic:tiny-llama-test", dtype="float32", device="cpu", data_parallel_size=2,
                            tensor_parallel_size=2)
    with pytest.raises(NotImplementedError):
        AsyncLLM(cfg)


def _dp_tp_worker(rank, world, out_dir):
    from litevllm_b200 import LLM, SamplingParams
    from litevllm_b200.parallel import state as pstate
    llm = LLM("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=4, max_model_len=128,
              data_parallel_size=2, tensor_parallel_size=2, comm_backend="nccl")
    st = pstate.get_state()
    prompts = [{"prompt_token_ids": [(5 * i + 3 * j) % 400 + 2 for i in range(9 + j)]} for j in range(5)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump({"tokens": [o.outputs[0].token_ids for o in outs], "replica": st.replica, "group_rank": st.rank,
                   "group_size": st.world_size, "served": llm.engine.stats()["observer"]["counters"]["requests_finished"]}, f)
    llm.shutdown()


def test_two_replicas_of_two_rank_tensor_parallel_groups():
    """Four ranks: replicas {0, 1} and {2, 3}, each a tensor-parallel pair.  Every rank returns all results in
    order, they equal the single-rank run, and each replica served only its share."""
    from litevllm_b200 import LLM, SamplingParams
    prompts = [{"prompt_token_ids": [(5 * i + 3 * j) % 400 + 2 for i in range(9 + j)]} for j in range(5)]
    ref = LLM("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=4, max_model_len=128)
    want = [o.outputs[0].token_ids for o in ref.generate(prompts, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))]
    ref.shutdown()
    with tempfile.TemporaryDirectory() as d:
        spawn(_dp_tp_worker, 4, args=(d,), port=29561)
        got = [json.load(open(os.path.join(d, f"rank{r}.json"))) for r in range(4)]
    assert all(g["tokens"] == want for g in got)
    assert [g["replica"] for g in got] == [0, 0, 1, 1] and [g["group_rank"] for g in got] == [0, 1, 0, 1]
    assert all(g["group_size"] == 2 for g in got)
    assert [g["served"] for g in got] == [3, 3, 2, 2]          # prompts 0, 2, 4 on replica 0; 1, 3 on replica 1
