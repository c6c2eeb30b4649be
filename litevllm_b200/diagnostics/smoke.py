"""Timed generation of one model with gates.

    python -m litevllm_b200.diagnostics.smoke --model synthetic:tiny-llama-test --device cpu --dtype float32 \\
        --prompt-length 32 --max-tokens 16 --repeat 2 --min-steady-decode-tps 1.5

Each repeat submits ``--batch`` random prompts of ``--prompt-length`` tokens through the engine's public
``add_request`` / ``step`` calls and reads the host clock at the first token of every request and at the end.
Steady-state decode speed excludes the first token of every request (it belongs to prefill) and the first
``--warmup-tokens`` decode steps.  The first repeat is the cold one (allocations, graph capture); the gates
``--min-cold-tps`` and ``--min-steady-decode-tps`` apply to the cold repeat and to the best warm repeat.
Exit status 1 when a gate fails.  Same role as tests/tools/run_deepseek_v4_flash_gpu_smoke.py of the reference
(arguments :54-79, steady-state definition :90-112).
"""
from __future__ import annotations

import argparse
import json
import os
import random
import sys
import time


def parse(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, help="checkpoint directory, GGUF file or synthetic:<preset>")
    ap.add_argument("--device", default="auto")
    ap.add_argument("--dtype", default="auto")
    ap.add_argument("--context-length", type=int, default=0, help="max_model_len (0: prompt + output + 8)")
    ap.add_argument("--prompt-length", type=int, default=32)
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--warmup-tokens", type=int, default=2)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--repeat", type=int, default=2)
    ap.add_argument("--min-cold-tps", type=float, default=0.0)
    ap.add_argument("--min-steady-decode-tps", type=float, default=0.0)
    ap.add_argument("--staging-budget-gb", type=float, default=0.0,
                    help="device budget for routed experts of GGUF MoE models (0: everything resident)")
    ap.add_argument("--full-resident", action="store_true", help="refuse a staging budget: all weights on the device")
    ap.add_argument("--no-graph", action="store_true", help="run without CUDA graphs")
    ap.add_argument("--profile-json", default="", help="write the result and the engine's statistics to this file")
    ap.add_argument("--seed", type=int, default=0)
    return ap.parse_args(argv)


def run(a) -> dict:
    if a.full_resident and a.staging_budget_gb > 0:
        raise SystemExit("--full-resident and --staging-budget-gb exclude each other")
    if a.staging_budget_gb > 0:
        os.environ["FI_EXPERT_STAGING_GB"] = repr(a.staging_budget_gb)
    elif a.full_resident:
        os.environ.pop("FI_EXPERT_STAGING_GB", None)
    from litevllm_b200 import LLM, SamplingParams
    kw = dict(device=a.device, dtype=a.dtype, max_num_seqs=max(1, a.batch),
              max_model_len=a.context_length or (a.prompt_length + a.max_tokens + 8 + 63) // 64 * 64)
    if a.no_graph:
        kw["enforce_eager"] = True
    llm = LLM(a.model, **kw)
    eng = llm.engine
    vocab = llm.vllm_config.model_config.arch.vocab_size
    rng = random.Random(a.seed)
    sp = SamplingParams(temperature=0.0, max_tokens=a.max_tokens, ignore_eos=True)
    sync = (lambda: None)
    if str(eng.device).startswith("cuda"):
        import torch
        sync = lambda: torch.cuda.synchronize(eng.device)      # noqa: E731
    repeats = []
    for r in range(a.repeat):
        prompts = [[rng.randrange(2, vocab) for _ in range(a.prompt_length)] for _ in range(a.batch)]
        sync()
        t0 = time.perf_counter()
        for i, p in enumerate(prompts):
            eng.add_request(f"smoke-{r}-{i}", {"prompt_token_ids": p}, sp)
        first, counts, marks = {}, {}, []
        while eng.has_unfinished_requests():
            outs = eng.step()
            sync()
            now = time.perf_counter()
            for o in outs:
                n = len(o.outputs[0].token_ids)
                if n and o.request_id not in first:
                    first[o.request_id] = now - t0
                counts[o.request_id] = n
            marks.append((now - t0, sum(counts.values())))
        total_s, total_tokens = marks[-1]
        t_first = max(first.values())
        # steady state: from the step that ended `warmup-tokens` decode steps after the last first token
        after = [m for m in marks if m[0] >= t_first]
        lo = after[min(a.warmup_tokens, len(after) - 1)]
        steady = (total_tokens - lo[1]) / (total_s - lo[0]) if total_s > lo[0] and total_tokens > lo[1] else 0.0
        repeats.append({"repeat": r, "cold": r == 0, "first_token_s": round(t_first, 4), "total_s": round(total_s, 4),
                        "generated_tokens": total_tokens, "tps_incl_prefill": round(total_tokens / total_s, 3),
                        "steady_decode_tps": round(steady, 3), "steady_tokens": total_tokens - lo[1]})
    warm = repeats[1:] or repeats
    result = {"model": a.model, "device": str(eng.device), "batch": a.batch, "prompt_length": a.prompt_length,
              "max_tokens": a.max_tokens, "repeats": repeats, "cold_tps": repeats[0]["tps_incl_prefill"],
              "steady_decode_tps": max(x["steady_decode_tps"] for x in warm),
              "cuda_graphs": bool(getattr(eng.model, "supports_cuda_graph", False)) and not a.no_graph,
              "expert_staging": eng.stats().get("expert_staging", {})}
    failures = []
    if result["cold_tps"] < a.min_cold_tps:
        failures.append(f"cold run {result['cold_tps']} tok/s < gate {a.min_cold_tps}")
    if result["steady_decode_tps"] < a.min_steady_decode_tps:
        failures.append(f"steady decode {result['steady_decode_tps']} tok/s < gate {a.min_steady_decode_tps}")
    result["failures"] = failures
    if a.profile_json:
        with open(a.profile_json, "w") as f:
            json.dump({"result": result, "engine": eng.stats()}, f, indent=1, default=str)
    llm.shutdown()
    return result


def main(argv=None) -> int:
    result = run(parse(argv))
    print(json.dumps(result))
    for msg in result["failures"]:
        print("GATE FAILED: " + msg, file=sys.stderr)
    return 1 if result["failures"] else 0


if __name__ == "__main__":
    sys.exit(main())
