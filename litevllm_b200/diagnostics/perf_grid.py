"""A grid of engine settings timed in interleaved rounds; with two points it is an A/B comparison.

    python -m litevllm_b200.diagnostics.perf_grid --model synthetic:tiny-llama-test \\
        --base '{"device": "cpu", "dtype": "float32"}' --set max_num_seqs=2,4 \\
        --tuning FASTINFERENCE_LITE_PREFILL_CHUNK=64,512 --batch 4 --prompt-length 64 --max-tokens 16 --rounds 3

Axes: ``--set name=v1,v2`` varies an engine argument, ``--tuning KEY=v1,v2`` a ``[tuning_keyvals]`` entry,
``--env NAME=v1,v2`` a process-environment switch of the kernel layer.  The grid is the product of all axes.
Every round times every point once, in an order rotated from round to round, so that clock and thermal drift
spread evenly over the points instead of favouring the one measured first; the report gives each point's median
tokens per second and its ratio to the first point.  Without ``--env`` all engines live in this process and are
built before the first round; environment switches are read when the package is imported, so an ``--env`` axis
runs every measurement as a child process (``litevllm_b200.diagnostics.smoke``), which also measures cold start.
Same role as tests/tools/perf_grid_search.py and interleaved_e2e_ab.py of the reference.
"""
from __future__ import annotations

import argparse
import itertools
import json
import os
import random
import statistics
import subprocess
import sys
import time


def _axis(spec: str) -> tuple[str, list[str]]:
    name, _, values = spec.partition("=")
    if not name or not values:
        raise SystemExit(f"axis {spec!r}: expected NAME=v1,v2,...")
    return name, values.split(",")


def _value(text: str):
    try:
        return json.loads(text)
    except ValueError:
        return text


def grid(sets, tunings, envs) -> list[dict]:
    axes = [("set", *_axis(s)) for s in sets] + [("tuning", *_axis(s)) for s in tunings] + [("env", *_axis(s)) for s in envs]
    points = []
    for combo in itertools.product(*[vals for _, _, vals in axes]):
        p = {"set": {}, "tuning": {}, "env": {}}
        for (kind, name, _), v in zip(axes, combo):
            p[kind][name] = _value(v) if kind == "set" else v
        p["label"] = " ".join(f"{n}={v}" for k in ("set", "tuning", "env") for n, v in p[k].items()) or "base"
        points.append(p)
    return points


def engine_kwargs(base: dict, point: dict, a) -> dict:
    kw = dict(base)
    kw.update(point["set"])
    kw.setdefault("max_num_seqs", a.batch)
    kw.setdefault("max_model_len", (a.prompt_length + a.max_tokens + 8 + 63) // 64 * 64)
    if point["tuning"]:
        fi = dict(kw.get("fastinference_config") or {})
        fi["tuning_keyvals"] = {**fi.get("tuning_keyvals", {}), **point["tuning"]}
        kw["fastinference_config"] = fi
    return kw


def _time_in_process(llm, prompts, max_tokens) -> float:
    from litevllm_b200 import SamplingParams
    sp = SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True)
    t0 = time.perf_counter()
    outs = llm.generate([{"prompt_token_ids": p} for p in prompts], sp)
    if str(llm.engine.device).startswith("cuda"):
        import torch
        torch.cuda.synchronize(llm.engine.device)
    dt = time.perf_counter() - t0
    return sum(len(o.outputs[0].token_ids) for o in outs) / dt


def _time_in_child(a, base: dict, point: dict) -> float:
    kw = engine_kwargs(base, point, a)
    extra = set(kw) - {"device", "dtype", "max_num_seqs", "max_model_len", "enforce_eager"}
    if extra:
        raise SystemExit(f"an --env axis runs child processes, which take device, dtype and the batch only; "
                         f"not {sorted(extra)}")
    cmd = [sys.executable, "-m", "litevllm_b200.diagnostics.smoke", "--model", a.model, "--device", str(kw.get("device", "auto")),
           "--dtype", str(kw.get("dtype", "auto")), "--batch", str(a.batch), "--prompt-length", str(a.prompt_length),
           "--max-tokens", str(a.max_tokens), "--repeat", "2", "--seed", str(a.seed)]
    if kw.get("enforce_eager"):
        cmd.append("--no-graph")
    env = dict(os.environ, **{k: str(v) for k, v in point["env"].items()})
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=a.child_timeout)
    if out.returncode not in (0, 1):
        raise RuntimeError(f"child failed for {point['label']}: {out.stderr[-400:]}")
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    return float(json.loads(line)["repeats"][-1]["tps_incl_prefill"])


def run(a) -> dict:
    base = json.loads(a.base)
    points = grid(a.set, a.tuning, a.env)
    if len(points) > a.max_points:
        raise SystemExit(f"{len(points)} grid points exceed --max-points {a.max_points}")
    child = any(p["env"] for p in points)
    rng = random.Random(a.seed)
    samples: list[list[float]] = [[] for _ in points]
    engines = []
    if not child:
        from litevllm_b200 import LLM
        engines = [LLM(a.model, **engine_kwargs(base, p, a)) for p in points]
        vocab = engines[0].vllm_config.model_config.arch.vocab_size
    try:
        for r in range(a.warmup_rounds + a.rounds):
            order = [(i + r) % len(points) for i in range(len(points))]
            prompts = None
            if not child:
                prompts = [[rng.randrange(2, vocab) for _ in range(a.prompt_length)] for _ in range(a.batch)]
            for i in order:
                tps = _time_in_child(a, base, points[i]) if child else _time_in_process(engines[i], prompts, a.max_tokens)
                if r >= a.warmup_rounds:
                    samples[i].append(tps)
    finally:
        for e in engines:
            e.shutdown()
    rows = []
    for p, s in zip(points, samples):
        rows.append({"label": p["label"], "set": p["set"], "tuning": p["tuning"], "env": p["env"],
                     "median_tps": round(statistics.median(s), 3), "min_tps": round(min(s), 3),
                     "max_tps": round(max(s), 3), "samples": len(s)})
    ref = rows[0]["median_tps"] or 1.0
    for row in rows:
        row["vs_first"] = round(row["median_tps"] / ref, 4)
    return {"model": a.model, "batch": a.batch, "prompt_length": a.prompt_length, "max_tokens": a.max_tokens,
            "rounds": a.rounds, "child_processes": child, "points": rows,
            "best": max(rows, key=lambda r: r["median_tps"])["label"]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--base", default="{}", help="engine arguments shared by all points, as JSON")
    ap.add_argument("--set", action="append", default=[], metavar="NAME=v1,v2")
    ap.add_argument("--tuning", action="append", default=[], metavar="KEY=v1,v2")
    ap.add_argument("--env", action="append", default=[], metavar="NAME=v1,v2")
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--prompt-length", type=int, default=64)
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--rounds", type=int, default=3)
    ap.add_argument("--warmup-rounds", type=int, default=1)
    ap.add_argument("--max-points", type=int, default=16)
    ap.add_argument("--child-timeout", type=float, default=900.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    rep = run(a)
    if a.json:
        print(json.dumps(rep))
    else:
        print(f"{'point':72s} {'median tok/s':>13s} {'min':>10s} {'max':>10s} {'vs first':>9s}")
        for r in rep["points"]:
            print(f"{r['label'][:72]:72s} {r['median_tps']:13.2f} {r['min_tps']:10.2f} {r['max_tps']:10.2f} {r['vs_first']:9.3f}")
        print("best: " + rep["best"])
    return 0


if __name__ == "__main__":
    sys.exit(main())
