"""Prompts with expectations, run greedily through the engine: a coarse check that a checkpoint still answers.

    python -m litevllm_b200.diagnostics.quality_spotcheck --model <m> --fixtures cases.json [--chat] [--min-pass-rate 0.9]

A fixture file is a JSON list of cases ``{"name", "prompt" | "messages", "max_tokens", "expect_any": [...],
"expect_all": [...], "expect_regex": "...", "forbid": [...]}``; matching is case-insensitive on the generated
text.  A case also fails on an empty answer, on a finish reason other than stop / length, and on degenerate
output (one token making up more than ``--max-repeat-share`` of an answer of 16 tokens or more), which is how
broken numerics usually show.  Exit status 1 when the pass rate is below ``--min-pass-rate``.  Same role as
tests/tools/quality_bar_spotcheck.py and gemma4_single_prompt_smoke.py of the reference.
"""
from __future__ import annotations

import argparse
import json
import re
import sys
from collections import Counter


def judge_case(case: dict, text: str, token_ids: list[int], finish_reason: str | None, max_repeat_share: float = 0.6) -> list[str]:
    """-> reasons the answer fails the case (empty: it passes)."""
    why = []
    low = text.lower()
    if not token_ids or not text.strip():
        why.append("empty answer")
    if finish_reason not in (None, "stop", "length"):
        why.append(f"finish reason {finish_reason}")
    if len(token_ids) >= 16:
        tok, n = Counter(token_ids).most_common(1)[0]
        if n / len(token_ids) > max_repeat_share:
            why.append(f"degenerate: token {tok} is {n} of {len(token_ids)} tokens")
    any_of = case.get("expect_any") or []
    if any_of and not any(s.lower() in low for s in any_of):
        why.append(f"none of {any_of} in the answer")
    for s in case.get("expect_all") or []:
        if s.lower() not in low:
            why.append(f"{s!r} missing")
    rx = case.get("expect_regex")
    if rx and not re.search(rx, text, flags=re.I | re.S):
        why.append(f"no match for /{rx}/")
    for s in case.get("forbid") or []:
        if s.lower() in low:
            why.append(f"forbidden {s!r} present")
    return why


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--fixtures", required=True)
    ap.add_argument("--engine", default="{}", help="engine arguments as JSON")
    ap.add_argument("--chat", action="store_true", help="render prompts through the tokenizer's chat template")
    ap.add_argument("--max-tokens", type=int, default=64, help="for cases that name none")
    ap.add_argument("--min-pass-rate", type=float, default=1.0)
    ap.add_argument("--max-repeat-share", type=float, default=0.6)
    a = ap.parse_args(argv)
    with open(a.fixtures) as f:
        cases = json.load(f)
    if not isinstance(cases, list) or not cases:
        print("error: the fixture file holds no cases", file=sys.stderr)
        return 2
    from litevllm_b200 import LLM, SamplingParams
    kw = {"max_num_seqs": min(8, len(cases))}
    kw.update(json.loads(a.engine))
    llm = LLM(a.model, **kw)
    try:
        tok = llm.get_tokenizer()
        prompts, params = [], []
        for c in cases:
            if "prompt_token_ids" in c:
                prompts.append({"prompt_token_ids": list(c["prompt_token_ids"])})
            else:
                msgs = c.get("messages") or [{"role": "user", "content": c["prompt"]}]
                if (a.chat or "messages" in c) and getattr(tok, "chat_template", None):
                    text = tok.apply_chat_template(msgs, tokenize=False, add_generation_prompt=True)
                else:
                    text = "\n".join(m["content"] for m in msgs)
                prompts.append(text)
            params.append(SamplingParams(temperature=0.0, max_tokens=int(c.get("max_tokens", a.max_tokens))))
        outs = llm.generate(prompts, params)
    finally:
        llm.shutdown()
    rows = []
    for c, o in zip(cases, outs):
        comp = o.outputs[0]
        why = judge_case(c, comp.text, list(comp.token_ids), comp.finish_reason, a.max_repeat_share)
        rows.append({"name": c.get("name", f"case{len(rows)}"), "passed": not why, "why": why,
                     "answer": comp.text[:200], "tokens": len(comp.token_ids)})
    rate = sum(r["passed"] for r in rows) / len(rows)
    print(json.dumps({"model": a.model, "cases": len(rows), "pass_rate": round(rate, 4), "results": rows}))
    for r in rows:
        if not r["passed"]:
            print(f"FAILED {r['name']}: " + "; ".join(r["why"]), file=sys.stderr)
    return 0 if rate >= a.min_pass_rate else 1


if __name__ == "__main__":
    sys.exit(main())
