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


def test_replicas_of_sharded_groups_are_refused():
    import pytest

    from litevllm_b200.config.parallel_config import ParallelConfig
    with pytest.raises(NotImplementedError):
        ParallelConfig.from_env(tp=2, dp=2)
