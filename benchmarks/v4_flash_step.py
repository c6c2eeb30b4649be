"""DeepSeek-V4-Flash-shaped steps on one GPU: the full-size layer geometry (hidden 4096, 64 heads over one
512-wide latent row, 256 experts of width 2048 with 6 per token, IQ2_XXS / Q2_K expert blocks, Q8_0
projections) with a configurable number of layers and random block weights.  Times a prefill chunk and decode
steps of the model-owned data plane with CUDA events and prints one JSON line (``FI_V4_DECODE_GRAPHS=0`` for
the decode step without its CUDA graphs).

    python benchmarks/v4_flash_step.py --layers 8 --batch 1 --prompt-len 64 --steps 16
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt-len", type=int, default=64)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--vocab", type=int, default=32768)
    ap.add_argument("--host-profile", action="store_true", help="print the host-side profile of extra decode steps")
    ap.add_argument("--kernel-table", action="store_true",
                    help="print the GPU kernels of one more prefill and one decode step by total time (shares only)")
    ap.add_argument("--staging-budget-gb", type=float, default=0.0,
                    help="device budget for routed experts; the rest stays in pinned host memory behind "
                         "least-recently-used slots (0: everything resident)")
    ap.add_argument("--pin-hot", type=int, default=0, help="after warm-up, pin this many most-used experts per block")
    ap.add_argument("--engine", action="store_true", help="also time LLM.generate of the same prompts (host clock)")
    a = ap.parse_args()
    if a.staging_budget_gb > 0:
        os.environ["FI_EXPERT_STAGING_GB"] = repr(a.staging_budget_gb)       # read when the model is built
    from litevllm_b200 import LLM
    from litevllm_b200.models.deepseek_v4_flash.model import BlockMatrix
    from litevllm_b200.models.presets import PRESETS
    PRESETS["v4-flash-shaped"] = {
        "architectures": ["DeepseekV4FlashForCausalLM"], "model_type": "deepseek_v4_flash", "hidden_size": 4096,
        "num_hidden_layers": a.layers, "num_attention_heads": 64, "num_key_value_heads": 1, "head_dim": 512,
        "qk_rope_head_dim": 64, "q_lora_rank": 1024, "sliding_window": 128, "index_n_heads": 64, "index_topk": 512,
        "hc_mult": 4, "o_groups": 8, "o_lora_rank": 1024, "n_routed_experts": 256, "num_experts_per_tok": 6,
        "moe_intermediate_size": 2048, "num_hash_layers": min(3, a.layers), "routed_scaling_factor": 1.5,
        "swiglu_limit": 10.0, "vocab_size": a.vocab, "rms_norm_eps": 1e-6, "max_position_embeddings": 4096,
        "intermediate_size": 2048, "eos_token_id": 1, "synthetic_block_weights": True,
    }
    llm = LLM("synthetic:v4-flash-shaped", device="cuda", max_model_len=max(256, a.prompt_len + a.steps + a.warmup + 8),
              max_num_seqs=max(8, a.batch))
    model = llm.engine.model
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(2, a.vocab, (a.prompt_len,), generator=g).tolist() for _ in range(a.batch)]

    def timed(fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(dev)
        e0.record()
        out = fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1), out

    model.prefill_request("warm", prompts[0][:16], 0, True)          # lazy allocations, kernel attributes
    model.release_request("warm")
    rids = [f"r{i}" for i in range(a.batch)]
    t_prefill, last, per_request = 0.0, [], []
    for rid, p in zip(rids, prompts):
        ms, tok = timed(lambda: model.prefill_request(rid, p, 0, True))
        t_prefill += ms
        per_request.append(round(ms, 1))
        last.append(tok)
    for _ in range(a.warmup):
        last = model.decode_tokens_batch(rids, last)
    if a.pin_hot > 0:
        from litevllm_b200.layers import expert_stager
        expert_stager.pin_hot_experts(model, a.pin_hot)

    def decode_steps():
        toks = last
        for _ in range(a.steps):
            toks = model.decode_tokens_batch(rids, toks)
        return toks

    t_decode, last = timed(decode_steps)
    ms_step = t_decode / a.steps
    if a.host_profile:
        import cProfile
        import pstats
        prof = cProfile.Profile()
        prof.enable()
        decode_steps()
        torch.cuda.synchronize(dev)
        prof.disable()
        pstats.Stats(prof, stream=sys.stderr).sort_stats("tottime").print_stats(28)
    rows_mb = round(model.request_bytes() / 2 ** 20, 2)
    if a.kernel_table:
        from torch.profiler import ProfilerActivity, profile
        for what, fn in (("prefill", lambda: model.prefill_request("kt", prompts[0], 0, True)), ("decode", decode_steps)):
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                fn()
                torch.cuda.synchronize(dev)
            print(f"--- {what}", file=sys.stderr)
            print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=14, max_name_column_width=60), file=sys.stderr)
        model.release_request("kt")
    engine = {}
    if a.engine:
        import time
        from litevllm_b200 import SamplingParams
        for rid in rids:
            model.release_request(rid)
        sp = SamplingParams(max_tokens=a.steps, temperature=0.0, ignore_eos=True)
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        outs = llm.generate([{"prompt_token_ids": p} for p in prompts], sp)
        dt = time.perf_counter() - t0
        n_out = sum(len(o.outputs[0].token_ids) for o in outs)
        engine = {"engine_generate_s": round(dt, 3), "engine_generated_tokens": n_out,
                  "engine_tok_s_incl_prefill": round(n_out / dt, 2)}
    weights = sum(p.numel() * p.element_size() for p in model.parameters())
    for layer in model.layers:
        weights += sum(v.numel() for v in layer.routed.raw.values()) if layer.routed is not None else 0
        if layer.routed is not None and layer.routed.stager is not None:
            weights += layer.routed.stager.device_bytes
        weights += sum(getattr(layer, n).nbytes() for n in model._LINEAR if isinstance(getattr(layer, n, None), BlockMatrix))
    weights += sum(m.nbytes() for m, _ in model._merged.values() if isinstance(m, BlockMatrix))
    print(json.dumps({
        "case": "v4_flash_shaped_step", "layers": a.layers, "batch": a.batch, "prompt_len": a.prompt_len,
        "prefill_ms_per_request": per_request,
        "prefill_ms_per_token": round(t_prefill / (a.batch * a.prompt_len), 3),
        "prefill_ms_per_token_per_layer": round(t_prefill / (a.batch * a.prompt_len * a.layers), 4),
        "decode_ms_per_step": round(ms_step, 3), "decode_ms_per_step_per_layer": round(ms_step / a.layers, 4),
        "decode_tok_s": round(a.batch * 1000.0 / ms_step, 2), "weights_gb": round(weights / 2 ** 30, 2),
        "rows_mb": rows_mb, **engine,
        "decode_graphs": os.environ.get("FI_V4_DECODE_GRAPHS", "1") != "0" and a.staging_budget_gb <= 0,
        "expert_staging": llm.engine.stats()["expert_staging"],
        "note": "model-owned data plane; per-layer figures scale to the 43 layers of the full model"}))


if __name__ == "__main__":
    main()
