"""One prefill step of the benchmark model (a micro-batch of whole prompts), bracketed by
cudaProfilerStart/Stop, for a per-kernel launch list:

    python benchmarks/prefill_step.py &&
    ncu --metrics gpu__time_duration.sum --clock-control none --profile-from-start off --csv \
        --log-file launches.csv python benchmarks/prefill_step.py

Without a profiler it prints the device time and the host wall time of the step (CUDA events / perf_counter)."""
from __future__ import annotations

import argparse
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tinyllama-1.1b")
    ap.add_argument("--prompts", type=int, default=8, help="prompts in the step (the engine's prefill micro-batch)")
    ap.add_argument("--prompt-len", type=int, default=1024)
    args = ap.parse_args()
    import torch

    from litevllm_b200 import LLM, SamplingParams
    B, P = args.prompts, args.prompt_len
    cfg = {"profile": "throughput", "tuning_keyvals": {"FASTINFERENCE_KV_MAX_ACTIVE_REQUESTS": str(B),
                                                       "FASTINFERENCE_LITE_PREFILL_MICROBATCH": str(B)}}
    llm = LLM(f"synthetic:{args.model}", dtype="bfloat16", max_num_seqs=B, max_model_len=P + 32,
              max_num_batched_tokens=max(8192, B * P), fastinference_config=cfg, device="cuda:0")
    eng = llm.engine
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(0, eng.arch.vocab_size, (B, P), generator=g).tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True)

    def one_pass(tag, profile):
        for i in range(B):
            eng.add_request(f"{tag}{i}", prompts[i], sp)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if profile:
            torch.cuda.profiler.start()
        t0 = time.perf_counter()
        e0.record()
        eng.step()                       # the prefill step of all B prompts
        e1.record()
        torch.cuda.synchronize()
        wall = (time.perf_counter() - t0) * 1e3
        if profile:
            torch.cuda.profiler.stop()
        while eng.has_unfinished_requests():
            eng.step()
        return e0.elapsed_time(e1), wall

    one_pass("warm", False)
    one_pass("warm2", False)
    dev_ms, wall_ms = one_pass("run", True)
    print(f"prefill step: {dev_ms:.3f} ms device time, {wall_ms:.3f} ms host wall time, {B} prompts x {P} tokens")
    import os
    os._exit(0)


if __name__ == "__main__":
    main()
