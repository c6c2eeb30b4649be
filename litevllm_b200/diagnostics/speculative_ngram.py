"""What prompt-lookup (n-gram) speculation would buy on a model's own greedy output.

    python -m litevllm_b200.diagnostics.speculative_ngram --model <m> --prompt-file prompts.json --max-tokens 256 -k 4

The engine generates greedily as usual.  The tool then replays every generated sequence: at each position a
proposer looks for the most recent earlier occurrence of the last 2..4 generated tokens in prompt + output and
proposes the ``k`` tokens that followed it; the proposal's longest prefix that equals what the model really
generated next is what a verify step would have accepted (greedy verification accepts exactly that prefix, plus
the one token the verify step computes itself).  Reported: proposals made, tokens accepted, tokens per verify
step, and the speed-up that follows for a given cost of a k-token verify step relative to a one-token step.
Nothing is changed in the engine; this is the measurement that decides whether speculation is worth building for
a workload.  Same role as tests/tools/gemma4_speculative_prototype.py of the reference.
"""
from __future__ import annotations

import argparse
import json
import sys


def propose(context: list[int], generated: int, k: int, ngram_min: int = 2, ngram_max: int = 4) -> list[int]:
    """Up to ``k`` draft tokens for ``context`` (prompt + output so far, of which the last ``generated`` are
    output): the continuation of the most recent earlier occurrence of the longest matching suffix."""
    for n in range(ngram_max, ngram_min - 1, -1):
        if generated < n or len(context) <= n:
            continue
        needle = context[-n:]
        for i in range(len(context) - n - 1, -1, -1):
            if context[i:i + n] == needle:
                return context[i + n:i + n + k]
    return []


def replay(prompt: list[int], output: list[int], k: int, ngram_min: int = 2, ngram_max: int = 4) -> dict:
    """Walk ``output`` as a speculative decoder would: each verify step yields the accepted draft prefix + 1."""
    pos, steps, proposed, accepted, with_draft = 0, 0, 0, 0, 0
    while pos < len(output):
        draft = propose(prompt + output[:pos], pos, k, ngram_min, ngram_max)
        hit = 0
        while hit < len(draft) and pos + hit < len(output) and draft[hit] == output[pos + hit]:
            hit += 1
        proposed += len(draft)
        accepted += hit
        with_draft += bool(draft)
        steps += 1
        pos += min(hit + 1, len(output) - pos)
    return {"tokens": len(output), "verify_steps": steps, "steps_with_draft": with_draft, "proposed": proposed,
            "accepted": accepted}


def summarise(parts: list[dict], verify_cost: float) -> dict:
    tot = {k: sum(p[k] for p in parts) for k in ("tokens", "verify_steps", "steps_with_draft", "proposed", "accepted")}
    steps = max(1, tot["verify_steps"])
    plain = tot["verify_steps"] - tot["steps_with_draft"]
    cost = plain + verify_cost * tot["steps_with_draft"]          # in units of one ordinary decode step
    tot.update(tokens_per_step=round(tot["tokens"] / steps, 4),
               acceptance=round(tot["accepted"] / tot["proposed"], 4) if tot["proposed"] else 0.0,
               projected_speedup=round(tot["tokens"] / cost, 4) if cost else 1.0, verify_cost=verify_cost)
    return tot


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--engine", default="{}", help="engine arguments as JSON")
    ap.add_argument("--prompt-file", default="", help="JSON list of prompts: strings or lists of token ids")
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("-k", type=int, default=4, help="draft tokens per proposal")
    ap.add_argument("--ngram-min", type=int, default=2)
    ap.add_argument("--ngram-max", type=int, default=4)
    ap.add_argument("--verify-cost", type=float, default=1.15,
                    help="cost of a verify step over k+1 positions relative to a one-token decode step")
    a = ap.parse_args(argv)
    from litevllm_b200 import LLM, SamplingParams
    if a.prompt_file:
        with open(a.prompt_file) as f:
            prompts = json.load(f)
    else:   # repetitive by construction, so that the default run shows a non-trivial acceptance
        prompts = [[(7 * i) % 23 + 5 for i in range(48)], [(3 * i) % 11 + 40 for i in range(32)]]
    kw = {"max_num_seqs": max(1, len(prompts))}
    kw.update(json.loads(a.engine))
    llm = LLM(a.model, **kw)
    try:
        tok = llm.get_tokenizer()
        ids = [p if isinstance(p, list) else tok.encode(p) for p in prompts]
        outs = llm.generate([{"prompt_token_ids": p} for p in ids],
                            SamplingParams(temperature=0.0, max_tokens=a.max_tokens, ignore_eos=False))
    finally:
        llm.shutdown()
    parts = [replay(p, list(o.outputs[0].token_ids), a.k, a.ngram_min, a.ngram_max) for p, o in zip(ids, outs)]
    rep = summarise(parts, a.verify_cost)
    rep["per_prompt"] = parts
    print(json.dumps(rep))
    return 0


if __name__ == "__main__":
    sys.exit(main())
