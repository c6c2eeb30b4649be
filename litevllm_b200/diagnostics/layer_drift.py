"""Per-layer hidden-state drift between two configurations of one model.

    python -m litevllm_b200.diagnostics.layer_drift --model synthetic:tiny-llama-test \\
        --b '{"device": "cpu", "dtype": "float32", "fastinference_config": {"kv_type": "fp8"}}'

Both configurations run the same prompt (prefill, then ``--decode-steps`` greedy steps that follow A's tokens so
the inputs stay identical).  Forward hooks on every decoder layer keep the layer's last-position output of each
step; the report gives, per step and layer, cosine similarity, relative L2 error and largest absolute difference
between A and B, names the first layer whose relative error exceeds ``--threshold``, and compares the final
tokens.  Exit status 1 when a layer exceeds the threshold.  Same role as
tests/tools/gemma4_layer_drift_diagnostic.py and gemma4_prefill_strict_audit.py of the reference.
"""
from __future__ import annotations

import argparse
import json
import re
import sys

import torch


def _layer_modules(model) -> list[tuple[str, torch.nn.Module]]:
    """The decoder layers: direct children of the model's longest ModuleList."""
    best: list[tuple[str, torch.nn.Module]] = []
    for name, mod in model.named_modules():
        if isinstance(mod, torch.nn.ModuleList) and len(mod) > len(best) and not re.search(r"vision|visual|tower", name):
            best = [(f"{name}.{i}", m) for i, m in enumerate(mod)]
    return best


class LayerTap:
    """Keeps, per forward call, the last row of every decoder layer's first floating-point output."""

    def __init__(self, model):
        self.layers = _layer_modules(model)
        self.calls: list[dict[str, torch.Tensor]] = []
        self._handles = []

    def _hook(self, name):
        def fn(_m, _inp, output):
            items = output if isinstance(output, (tuple, list)) else (output,)
            # a layer that returns (hidden, residual) is judged by their sum: the stream the next layer reads
            floats = [t for t in items if isinstance(t, torch.Tensor) and t.is_floating_point() and t.dim() >= 2]
            if not floats:
                return
            t = floats[0] if len(floats) == 1 or floats[0].shape != floats[1].shape else floats[0] + floats[1]
            row = t.detach().reshape(-1, t.shape[-1])[-1].float().cpu().clone()     # a copy: the stream is updated in place
            if not self.calls or name in self.calls[-1]:
                self.calls.append({})
            self.calls[-1][name] = row
        return fn

    def __enter__(self):
        for name, mod in self.layers:
            self._handles.append(mod.register_forward_hook(self._hook(name)))
        return self

    def __exit__(self, *exc):
        for h in self._handles:
            h.remove()
        self._handles.clear()
        return False


def trace(model_name: str, kwargs: dict, prompt: list[int], steps: int, follow: list[int] | None):
    """-> (per-call layer rows, generated tokens).  ``follow``: tokens to feed instead of the model's own."""
    from litevllm_b200 import LLM, SamplingParams
    kw = dict(max_num_seqs=1, max_model_len=(len(prompt) + steps + 8 + 63) // 64 * 64, enforce_eager=True)
    kw.update(kwargs)
    llm = LLM(model_name, **kw)
    calls, tokens = [], []
    try:
        with LayerTap(llm.engine.model) as tap:
            if not tap.layers:
                raise SystemExit("this model keeps its layers outside a module list: nothing to tap")
            cur = list(prompt)
            for s in range(steps + 1):
                # one request per step with the prefix so far: identical inputs for A and B at every step
                before = len(tap.calls)
                out = llm.generate([{"prompt_token_ids": cur}], SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True))
                tok = out[0].outputs[0].token_ids[0]
                tokens.append(tok)
                calls.append(tap.calls[-1] if len(tap.calls) > before else {})
                cur = cur + [follow[s] if follow is not None and s < len(follow) else tok]
    finally:
        llm.shutdown()
    return calls, tokens


def compare(a_calls, b_calls, threshold: float) -> dict:
    rows, first_bad = [], None
    for step, (ca, cb) in enumerate(zip(a_calls, b_calls)):
        for name in ca:
            if name not in cb:
                continue
            x, y = ca[name], cb[name]
            diff = (x - y)
            rel = float(diff.norm() / x.norm().clamp_min(1e-12))
            cos = float(torch.nn.functional.cosine_similarity(x, y, dim=0))
            row = {"step": step, "layer": name, "cosine": round(cos, 6), "rel_l2": round(rel, 6),
                   "max_abs": round(float(diff.abs().max()), 6), "finite": bool(torch.isfinite(y).all())}
            rows.append(row)
            if first_bad is None and (rel > threshold or not row["finite"]):
                first_bad = row
    return {"rows": rows, "first_over_threshold": first_bad,
            "worst": max(rows, key=lambda r: r["rel_l2"]) if rows else None}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--a", default='{"device": "cpu", "dtype": "float32"}', help="engine arguments of A as JSON")
    ap.add_argument("--b", required=True, help="engine arguments of B as JSON")
    ap.add_argument("--prompt-length", type=int, default=24)
    ap.add_argument("--decode-steps", type=int, default=4)
    ap.add_argument("--threshold", type=float, default=0.05, help="relative L2 error that counts as drift")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    import random
    rng = random.Random(a.seed)
    prompt = [rng.randrange(2, 200) for _ in range(a.prompt_length)]
    a_calls, a_tokens = trace(a.model, json.loads(a.a), prompt, a.decode_steps, None)
    b_calls, b_tokens = trace(a.model, json.loads(a.b), prompt, a.decode_steps, a_tokens)
    rep = compare(a_calls, b_calls, a.threshold)
    rep.update(tokens_a=a_tokens, tokens_b=b_tokens,
               tokens_agree=sum(x == y for x, y in zip(a_tokens, b_tokens)), threshold=a.threshold)
    if a.json:
        print(json.dumps(rep))
    else:
        print(f"{'step':>4s} {'layer':32s} {'cosine':>10s} {'rel_l2':>10s} {'max_abs':>10s}")
        for r in rep["rows"]:
            print(f"{r['step']:4d} {r['layer'][:32]:32s} {r['cosine']:10.6f} {r['rel_l2']:10.6f} {r['max_abs']:10.6f}")
        print(f"tokens agree at {rep['tokens_agree']} of {len(a_tokens)} steps: A {a_tokens}  B {b_tokens}")
        bad = rep["first_over_threshold"]
        print("no layer over the threshold" if bad is None else
              f"first drift: step {bad['step']} {bad['layer']} rel_l2 {bad['rel_l2']} (threshold {a.threshold})")
    return 0 if rep["first_over_threshold"] is None else 1


if __name__ == "__main__":
    sys.exit(main())
