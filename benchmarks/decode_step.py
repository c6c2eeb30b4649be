"""A few pipelined decode steps of the benchmark model, bracketed by cudaProfilerStart/Stop, for a
per-kernel launch list of one captured decode step:

    python benchmarks/decode_step.py --steps 2 &&
    ncu --metrics gpu__time_duration.sum --clock-control none --profile-from-start off --csv \
        --log-file launches.csv python benchmarks/decode_step.py --steps 2

Without a profiler it prints the device time per step (CUDA events)."""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tinyllama-1.1b")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=2)
    args = ap.parse_args()
    import torch

    from litevllm_b200 import LLM, SamplingParams
    B, P = args.batch, args.prompt_len
    cfg = {"profile": "throughput", "tuning_keyvals": {"FASTINFERENCE_KV_MAX_ACTIVE_REQUESTS": str(B),
                                                       "FASTINFERENCE_LITE_PREFILL_MICROBATCH": "8"}}
    llm = LLM(f"synthetic:{args.model}", dtype="bfloat16", max_num_seqs=B, max_model_len=P + 64,
              max_num_batched_tokens=max(8192, B * P), fastinference_config=cfg, device="cuda:0")
    eng = llm.engine
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(0, eng.arch.vocab_size, (B, P), generator=g).tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)
    for i in range(B):
        eng.add_request(f"r{i}", prompts[i], sp)
    while any(eng.scheduler.requests[f"r{i}"].is_prefill for i in range(B)):
        eng.step()
    for _ in range(6):
        eng.step()                      # captures the decode graph, settles the pipeline
    pipe = eng.backend.pipeline
    while pipe.inflight:
        pipe.collect_oldest()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()
    e0.record()
    for _ in range(args.steps):
        pipe.launch(read_back=False)
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print(f"decode step: {e0.elapsed_time(e1) / args.steps:.4f} ms device time, batch {B}, context {P + 8}")
    import os
    os._exit(0)


if __name__ == "__main__":
    main()
