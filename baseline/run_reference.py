"""Reference arm of ``bench.py``: runs the unmodified reference project from ``baseline/_ref`` in a
child process (so that ``import vllm`` resolves to it and none of this repository's engine is
loaded) and relays its JSON line.  Install once with::

    python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse \
        --target baseline/_ref <reference checkout>
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"


def unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why}


def run_reference_bench(args, metric: str, baseline_tps: float) -> dict:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if args.gpus > 1 or world > 1:
        # single-GPU engine: device hard-wired to cuda:0, no collective or process-group code
        return unavailable("the reference is a single-GPU engine (no distributed layer); "
                           "only --gpus 1 can be measured") if rank == 0 else {}
    if not (REF_DIR / "vllm" / "__init__.py").is_file():
        return unavailable("baseline/_ref is not installed (pip install --target baseline/_ref of the reference)")
    env = dict(os.environ)
    env["PYTHONPATH"] = str(REF_DIR) + os.pathsep + env.get("PYTHONPATH", "")
    env.pop("FASTINFERENCE_CONFIG", None)
    cmd = [sys.executable, str(HERE / "ref_child.py"), "--ref-dir", str(REF_DIR), "--steps", str(args.steps),
           "--warmup", str(args.warmup), "--batch", str(args.batch), "--prompt-len", str(args.prompt_len)]
    try:
        proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1500, cwd="/tmp")
    except subprocess.TimeoutExpired:
        return unavailable("reference run did not finish within 1500 s")
    line = next((l for l in proc.stdout.splitlines()[::-1] if l.startswith("REFJSON ")), None)
    if proc.returncode != 0 or line is None:
        tail = (proc.stderr or proc.stdout).strip().splitlines()[-3:]
        return unavailable("reference run failed: " + " | ".join(t.strip()[:200] for t in tail))
    res = json.loads(line[len("REFJSON "):])
    res["metric"] = metric
    res["higher_is_better"] = True
    res["scaling"] = "strong"
    res["vs_baseline"] = round(res["value"] / baseline_tps, 2)
    # the reference's timed loop IS its public API (LiteEngine.add_request + LiteEngine.step with host-side
    # token lists in and sampled ids out), so its end-to-end figure is the same measurement
    res.setdefault("e2e", {"value": res["value"], "unit": res.get("unit", "tok/s"),
                           "api": "reference LiteEngine.add_request + LiteEngine.step",
                           "h2d_bytes_per_step": None, "d2h_bytes_per_step": None})
    return res
