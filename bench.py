"""Headline benchmark: decode tokens/s (aggregate over the batch) and p50 time-to-first-token for
a TinyLlama-1.1B-shaped decoder in bf16, batch 32, prompt 1024 (+ up to 1024 generated tokens),
random-init weights, uniform-random prompt token ids.

One "step" = one decode step of the whole batch (32 new tokens).  After the prefill and W untimed
warm-up steps, exactly K steps are timed twice:
  * ``value``  : device-timed (CUDA events) replay of the engine's decode step with the sampled token
                 fed back on the device (kernel-only view);
  * ``e2e``    : the same K steps driven through the public engine API (``add_request`` + ``step``),
                 where every step copies its inputs (token ids + batch metadata) from pinned host
                 memory to the device and reads the sampled tokens back to the host.
Multi-GPU (``--gpus N`` under torchrun): tensor parallel over N ranks, one process per GPU; times
are the max over ranks.  ``--impl reference`` runs the unmodified reference project instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

BASELINE_TPS = 542.4   # reference README: TinyLlama-1.1B bf16, BS=32, 2048 ctx, aggregate tok/s (Radeon 8060S)
# published reference numbers per benchmark model (tok/s on the reference's own hardware), for vs_baseline
PUBLISHED_TPS = {"tinyllama-1.1b": 542.4,        # aggregate, batch 32
                 "dense-9b-awq": 205.1,          # Qwen3.5-9B AWQ int4, batch 16, aggregate
                 "gemma4-26b-a4b": 12.39,        # decode tok/s at batch 1
                 "deepseek-mla-moe": 1.78,       # DeepSeek-V4-Flash Q2 GGUF decode tok/s at batch 1
                 "deepseek-v4-flash": 1.78}      # the same published figure: this preset has that file's geometry
METRIC = "decode tok/s aggregate + p50 TTFT at 1/2/4/8 B200, device-timed max over ranks"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="tinyllama-1.1b")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--comm-backend", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--parallel", default="auto", choices=["auto", "dp", "tp", "ep", "tpep"],
                    help="how N GPUs are used: dp = N whole-engine replicas with the batch sharded over them, tp = "
                         "tensor parallel with the fused collectives, ep = expert parallel (MoE models: experts sharded, "
                         "attention replicated), tpep = experts sharded and attention / dense layers tensor parallel; auto = dp "
                         "for the headline model when N divides the batch (a 1.1B model at batch 32 is bound by "
                         "per-kernel latency, so replicas beat sharding), else tp")
    ap.add_argument("--profile-json", default=None, help="write per-phase timings here")
    ap.add_argument("--ctx-points", type=int, nargs="*", default=[1536, 2040],
                    help="contexts at which the K decode steps are timed again (headline model only)")
    ap.add_argument("--no-extra-configs", dest="extra_configs", action="store_false",
                    help="skip the short runs of the other BASELINE configurations (one-GPU runs only)")
    ap.add_argument("--extra-budget-s", type=float, default=240.0,
                    help="no further extra configuration is started once this much time went into them")
    ap.add_argument("--no-check-tokens", dest="check_tokens", action="store_false",
                    help="multi-GPU runs: skip the one-GPU reference pass that the first tokens are compared with")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi every 20 ms from before the warm-up until
    after the last timed region.  ``mark()`` brackets a region by host time so the samples that fell
    inside it can be reported separately from the samples of the whole run under load."""
    QUERY = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = Path(f"/tmp/fi_bench_clocks_{os.getpid()}.csv")
        self.rows: list | None = None

    def start(self):
        try:
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.gpu_index)], stdout=self.fh, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> None:
        import datetime
        self.rows = []
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.fh.close()
        for line in self.path.read_text().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 10:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                sm, mx, pw = float(parts[2]), float(parts[3]), float(parts[4])
            except ValueError:
                continue
            active = [n for n, v in zip(self.NAMES, parts[6:10]) if v.lower().startswith("active")]
            self.rows.append((ts, sm, mx, pw, active))
        try:
            self.path.unlink()
        except OSError:
            pass

    def summary(self, t0: float | None = None, t1: float | None = None, min_power_w: float = 0.0) -> dict:
        """Median SM clock / max clock / throttle reasons of the samples in [t0, t1] (epoch seconds;
        None = the whole recording), optionally only samples drawing at least ``min_power_w``."""
        if self.rows is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        sel = [r for r in self.rows if (t0 is None or r[0] >= t0 - 0.02) and (t1 is None or r[0] <= t1 + 0.02)
               and r[3] >= min_power_w]
        reasons = sorted({n for r in sel for n in r[4]})
        return {"sm_mhz": statistics.median(r[1] for r in sel) if sel else None,
                "sm_max_mhz": max(r[2] for r in sel) if sel else None,
                "power_w_max": max(r[3] for r in sel) if sel else None,
                "samples": len(sel), "reasons": reasons}


def _token_hash(rows) -> str:
    import hashlib
    h = hashlib.sha1()
    for r in rows:
        h.update((",".join(str(int(t)) for t in r) + ";").encode())
    return h.hexdigest()[:16]


def _build_llm(args, world: int, local_rank: int, tp: int, ep: int, max_len: int, model: str | None = None,
               batch: int | None = None, prompt_len: int | None = None, extra_cfg: dict | None = None, dp: int = 1):
    from litevllm_b200 import LLM
    B = batch or args.batch
    P = prompt_len or args.prompt_len
    cfg = {"profile": "throughput",
           "tuning_keyvals": {"FASTINFERENCE_GPU_GREEDY_SAMPLING": "0",
                              "FASTINFERENCE_KV_MAX_ACTIVE_REQUESTS": str(B),
                              "FASTINFERENCE_LITE_PREFILL_MICROBATCH": "8"}}
    if extra_cfg:
        cfg.update(extra_cfg)
    return LLM(f"synthetic:{model or args.model}", dtype="bfloat16", max_num_seqs=B, max_model_len=max_len,
               max_num_batched_tokens=max(8192, B * P), tensor_parallel_size=tp, expert_parallel_size=ep,
               data_parallel_size=dp, comm_backend=args.comm_backend, fastinference_config=cfg, device=f"cuda:{local_rank}")


def _greedy_tokens(eng, prompts, n_new: int, tag: str, first_logits: dict | None = None):
    """First ``n_new`` greedy tokens of every prompt through the public engine API.  ``first_logits``
    (optional dict) receives the logits row each request's first token was sampled from (prompt index ->
    fp32 CPU tensor), tapped where the backend hands the prefill logits to the sampler."""
    from litevllm_b200 import SamplingParams
    sp = SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True)
    got = {}
    backend = eng.backend
    orig_sample = backend._sample
    if first_logits is not None:
        def tapped(logits, reqs):
            for row, st in zip(logits, reqs):
                if st.request_id.startswith(tag + "-") and st.num_generated == 0:
                    first_logits.setdefault(int(st.request_id[len(tag) + 1:]), row.detach().float().cpu())
            return orig_sample(logits, reqs)
        backend._sample = tapped
    try:
        for i, p in enumerate(prompts):
            eng.add_request(f"{tag}-{i}", p, sp)
        while eng.has_unfinished_requests():
            for o in eng.step():
                if o is not None and o.finished:
                    got[o.request_id] = list(o.outputs[0].token_ids)
    finally:
        if first_logits is not None:
            backend._sample = orig_sample
    return [got[f"{tag}-{i}"] for i in range(len(prompts))]


def _short_config_runs(args, local_rank: int, model: str, batches: list[int], prompt_len: int, new_tokens: int) -> list:
    """Short own-arm runs of another BASELINE configuration on one GPU, one engine for all batch sizes:
    p50 TTFT of the batch and the device-timed decode rate over ``new_tokens - 4`` pipelined steps."""
    import gc

    import torch
    from litevllm_b200 import SamplingParams
    t_build = time.perf_counter()
    bmax = max(batches)
    llm = _build_llm(args, 1, local_rank, 1, 1, (prompt_len + new_tokens + 32 + 15) // 16 * 16, model=model,
                     batch=bmax, prompt_len=prompt_len)
    eng = llm.engine
    build_s = time.perf_counter() - t_build
    out = []
    try:
        g = torch.Generator().manual_seed(4321)
        ids = torch.randint(0, eng.arch.vocab_size, (bmax, prompt_len), generator=g, dtype=torch.int64).pin_memory()
        for batch in batches:
            prompts = [r.tolist() for r in ids[:batch]]
            _greedy_tokens(eng, prompts, 4, f"cfgwarm{batch}")     # same shapes as the timed pass: graphs, scratch, attributes
            torch.cuda.synchronize()
            sp = SamplingParams(temperature=0.0, max_tokens=new_tokens, ignore_eos=True)
            t0 = time.perf_counter()
            for i, p in enumerate(prompts):
                eng.add_request(f"cfg{batch}-{i}", p, sp)
            ttft = {}
            while len(ttft) < batch:
                outs = eng.step()
                now = time.perf_counter()
                for o in outs:
                    if o is not None and o.request_id not in ttft:
                        ttft[o.request_id] = now - t0
            eng.step()
            torch.cuda.synchronize()
            steps = max(1, new_tokens - 4)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            n_tok = 0
            for _ in range(steps):
                n_tok += len(eng.step())
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            while eng.has_unfinished_requests():
                eng.step()
            out.append({"model": model, "batch": batch, "prompt_len": prompt_len, "new_tokens": new_tokens,
                        "decode_tok_s": round(n_tok / (ms / 1e3), 1), "ms_per_step": round(ms / steps, 3),
                        "timed_steps": steps, "tokens_in_timed_region": n_tok,
                        "ttft_p50_ms": round(statistics.median(ttft.values()) * 1e3, 1),
                        "kv_cache": str(eng.kv_plan.dtype), "build_s": round(build_s, 1),
                        "published_reference_tok_s": PUBLISHED_TPS.get(model)})
    finally:
        llm.shutdown()
        del llm, eng
        gc.collect()
        torch.cuda.empty_cache()
    return out


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist

    from litevllm_b200 import SamplingParams, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torchrun for N>1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    B, P, K, W = args.batch, args.prompt_len, args.steps, args.warmup
    mode = args.parallel
    if mode == "auto":
        mode = "dp" if (world > 1 and args.model == "tinyllama-1.1b" and B % world == 0) else "tp"
    if mode == "dp" and B % world != 0:
        raise SystemExit(f"--parallel dp shards the batch: {B} requests do not divide over {world} replicas")
    # requests this rank serves itself: all of them, or its share when the ranks are replicas
    mine = list(range(rank, B, world)) if mode == "dp" else list(range(B))
    Bl = len(mine)
    slack = (Bl + 7) // 8 + 2         # decode steps early finishers of the prefill run ahead
    ctx_points = [c for c in args.ctx_points if c > P + 8] if args.model == "tinyllama-1.1b" else []
    max_len = max([P + 1 + W + K + slack + 16] + [c + W + K + slack + 8 for c in ctx_points])
    max_len = (max_len + 15) // 16 * 16
    sampler = ClockSampler(local_rank)
    sampler.start()

    g = torch.Generator().manual_seed(1234)
    vocab_guess = None
    N_CHECK = 16

    # ------------------------------------------------------------------ TP=1 reference tokens (multi-GPU runs)
    # Every rank runs the same prompts through a one-GPU engine on its own GPU before the parallel engine exists;
    # the parallel run's first tokens are compared with rank 0's.  All ranks do it, not only rank 0: a rank that
    # skipped this pass would enter the first parallel step with cold kernels (lazy module loads, attribute
    # set-up) and fall behind the warm rank by more than the one-second budget of the in-kernel peer waits.
    tp1_tokens = None
    if world > 1 and args.check_tokens:
        # replicas serve their own share of the prompts at their own batch size: the reference pass does the same,
        # so that both walk through identical kernels and the tokens can be compared bit for bit
        shard = mine if mode == "dp" else list(range(B))
        llm1 = _build_llm(args, 1, local_rank, 1, 1, max_len, batch=len(shard))
        vocab1 = llm1.engine.arch.vocab_size
        g1 = torch.Generator().manual_seed(1234)
        ids1 = torch.randint(0, vocab1, (B, P), generator=g1, dtype=torch.int64)
        tp1_logits = {}
        shard_tokens = _greedy_tokens(llm1.engine, [ids1[i].tolist() for i in shard], N_CHECK, "tp1", tp1_logits)
        tp1_tokens = None
        if rank == 0:        # indexed by prompt number, like the run that follows
            tp1_tokens = {i: shard_tokens[k] for k, i in enumerate(shard)}
            tp1_logits = {i: tp1_logits[k] for k, i in enumerate(shard) if k in tp1_logits}
        llm1.shutdown()
        del llm1
        import gc
        gc.collect()
        torch.cuda.empty_cache()

    if args.profile_json:
        from litevllm_b200.utils.profiling import PROFILER
        PROFILER.configure(True, nvtx=True)      # event pairs are resolved after the timed regions
    tp = world if mode in ("tp", "tpep") else 1
    ep = world if mode in ("ep", "tpep") else 1
    llm = _build_llm(args, world, local_rank, tp, ep, max_len, batch=Bl, dp=world if mode == "dp" else 1)
    eng = llm.engine
    vocab = eng.arch.vocab_size
    # prompts live in pinned host memory; the engine's batch builder copies them to the device
    prompt_ids = torch.randint(0, vocab, (B, P), generator=g, dtype=torch.int64).pin_memory()
    prompts = [prompt_ids[i].tolist() for i in mine]
    sp = SamplingParams(temperature=0.0, max_tokens=1 + W + K + slack, ignore_eos=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ------------------------------------------------------------------ warm-up at the timed shapes
    # All B prompts, full length: the prefill kernels, the bucket-B decode graph, every lazily sized
    # scratch buffer and kernel attribute exist before any clock starts.  The tokens double as the
    # parity check against the one-GPU run.
    run_logits = {} if (tp1_tokens is not None and rank == 0) else None
    first_tokens = _greedy_tokens(eng, prompts, N_CHECK, "warm", run_logits)
    barrier()
    tokens_match = None
    tokens_check = None
    if tp1_tokens is not None and rank == 0:
        tp1_tokens = [tp1_tokens[i] for i in mine]
        tp1_logits = {k: tp1_logits[i] for k, i in enumerate(mine) if i in tp1_logits}
        # 16 greedy tokens per prompt, strictly; and, because random-init logits are nearly flat and the
        # parallel run sums in another order, the first token again with near-ties set aside: a prompt
        # counts as a near-tie when the one-GPU run's top-2 margin is below four times the largest
        # logit difference seen between the two runs
        tokens_match = _token_hash(tp1_tokens) == _token_hash(first_tokens)
        first_equal = [int(a[0] == b[0]) for a, b in zip(tp1_tokens, first_tokens)]
        tokens_check = {"prompts": Bl, "tokens_per_prompt": N_CHECK, "first_token_equal": sum(first_equal),
                        "hash_tp1": _token_hash(tp1_tokens), "hash_this_run": _token_hash(first_tokens)}
        common = [i for i in range(Bl) if i in tp1_logits and i in run_logits
                  and tp1_logits[i].shape == run_logits[i].shape]
        if common:
            diff = max(float((tp1_logits[i] - run_logits[i]).abs().max()) for i in common)
            top2 = {i: torch.topk(tp1_logits[i], 2).values for i in common}
            margin = {i: float(top2[i][0] - top2[i][1]) for i in common}
            clear = [i for i in common if margin[i] > 4.0 * diff]
            tokens_check.update({
                "logits_max_abs_diff": round(diff, 5),
                "logits_abs_max": round(max(float(tp1_logits[i].abs().max()) for i in common), 4),
                "prompts_with_clear_winner": len(clear),
                "first_token_equal_where_clear": sum(first_equal[i] for i in clear),
                "first_token_match_outside_near_ties": all(first_equal[i] for i in clear)})

    # ------------------------------------------------------------------ e2e: public API, H2D + D2H each step
    def submit_and_first_tokens(tag: str, params) -> list[float]:
        t_submit = time.perf_counter()
        for i in range(Bl):
            eng.add_request(f"{tag}-{i}", prompts[i], params)
        seen = {}
        while len(seen) < Bl:
            outs = eng.step()
            now = time.perf_counter()
            for o in outs:
                if o is not None and o.request_id not in seen:
                    seen[o.request_id] = now - t_submit
        return list(seen.values())

    # first submission: TTFT only (two tokens per request, then it drains)
    ttft_a = submit_and_first_tokens("ttfta", SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
    while eng.has_unfinished_requests():
        eng.step()
    barrier()
    ttft_b = submit_and_first_tokens("e2e", sp)                # second submission: TTFT, then the timed decode
    for _ in range(W):
        eng.step()
    barrier()
    launches0 = ops.launch_count()
    replays0 = eng.decode_executor.graph_replays
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.time()
    h0 = time.perf_counter()
    ev0.record()
    n_tokens = 0
    for _ in range(K):
        outs = eng.step()
        n_tokens += len(outs)
    ev1.record()
    torch.cuda.synchronize()
    e2e_wall_ms = max_over_ranks((time.perf_counter() - h0) * 1e3)
    wall1 = time.time()
    barrier()
    e2e_ms = max_over_ranks(ev0.elapsed_time(ev1))
    e2e_window = (wall0, wall1)
    assert n_tokens == Bl * K, f"expected {Bl * K} tokens in the timed region, got {n_tokens}"
    while eng.has_unfinished_requests():
        eng.step()
    ttft_runs = [max_over_ranks(statistics.median(t) * 1e3) for t in (ttft_a, ttft_b)]
    ttft_p50_ms = max_over_ranks(statistics.median(ttft_a + ttft_b) * 1e3)
    bucket = eng.builder.bucket_for(Bl)
    copies = world if mode == "dp" else 1               # every replica copies its own metadata and token ids
    h2d_per_step = 4 * bucket * 4 * copies              # 4 x int32 metadata rows (positions, slots, lengths, slot ids); token ids stay on the device
    d2h_per_step = Bl * 8 * copies                       # sampled token ids (int64)

    # ------------------------------------------------------------------ device-only: decode steps back to back
    # Same engine, same captured graph: the decode pipeline is driven directly, sampled tokens are fed
    # back on the device and nothing is read back or post-processed on the host inside the timed region.
    sp_long = SamplingParams(temperature=0.0, max_tokens=max_len - P - 2, ignore_eos=True)
    for i in range(Bl):
        eng.add_request(f"dev-{i}", prompts[i], sp_long)
    while any(eng.scheduler.requests[f"dev-{i}"].is_prefill for i in range(Bl)):
        eng.step()
    for _ in range(W):
        eng.step()
    pipe = eng.backend.pipeline
    assert pipe is not None and pipe.active and len(pipe.reqs) == Bl, "decode pipeline not active"
    while pipe.inflight:           # settle the step launched by the warm-up
        pipe.collect_oldest()

    def timed_device_steps() -> tuple[float, tuple[float, float], int, int]:
        barrier()
        r0, l0 = eng.decode_executor.graph_replays, ops.launch_count()
        w0 = time.time()
        ev0.record()
        for _ in range(K):
            pipe.launch(read_back=False)
        ev1.record()
        barrier()
        w1 = time.time()
        return (max_over_ranks(ev0.elapsed_time(ev1)), (w0, w1), eng.decode_executor.graph_replays - r0,
                ops.launch_count() - l0)

    dev_ms, dev_window, dev_replays, dev_eager = timed_device_steps()
    ctx_start = int(pipe.pos.max()) - K

    # the same K steps at longer contexts: positions jump ahead (the KV blocks in between are allocated and
    # zero-filled, not computed and not timed), W warm-up steps, then K timed steps
    by_ctx = {str(ctx_start): round(dev_ms / K, 4)}
    for ctx in ctx_points:
        cur = int(pipe.pos.max())
        if ctx <= cur or ctx + W + K + 2 >= max_len:
            continue
        while pipe.inflight:
            pipe.collect_oldest()
        torch.cuda.synchronize()
        delta = ctx - cur
        for st in pipe.reqs:
            old_blocks = len(eng.backend.kv.blocks_of(st.request_id))
            eng.backend.kv.ensure_blocks(st.request_id, st.seq_len + delta + 1)
            fresh = eng.backend.kv.blocks_of(st.request_id)[old_blocks:]
            if fresh:
                idx = torch.tensor(fresh, device=dev, dtype=torch.int64)
                for kc, vc in eng.kv_cache.layers:
                    kc.index_fill_(0, idx, 0)
                    vc.index_fill_(0, idx, 0)
            st.seq_len += delta
        pipe.pos = pipe.pos + delta
        pipe._first = True
        for _ in range(W):
            pipe.launch(read_back=False)
        ms_c, _, _, _ = timed_device_steps()
        by_ctx[str(ctx)] = round(ms_c / K, 4)

    # diagnostic only (not a valid decode: the inputs do not advance): the captured step replayed back
    # to back with no host work in between = the pure GPU time of one step
    entry = eng.decode_executor._graphs.get((bucket, True))
    graph_only_ms = None
    if entry is not None and world == 1:
        gr = entry[0]
        torch.cuda.synchronize()
        ev0.record()
        for _ in range(32):
            gr.replay()
        ev1.record()
        torch.cuda.synchronize()
        graph_only_ms = ev0.elapsed_time(ev1) / 32
    while pipe.inflight:
        pipe.collect_oldest()
    pipe.stop()
    for i in range(Bl):
        eng.abort_request(f"dev-{i}")
    ops.check_status(dev)
    per_graph = getattr(eng.decode_executor, "launches_per_graph", {}).get(bucket, 0)
    sampler.stop()

    from litevllm_b200.parallel import state as pstate
    pst = pstate.get_state()
    effective_backend = "none (one GPU)" if world == 1 else pst.comm_backend
    if mode == "dp" and world > 1:
        effective_backend = "none (replicas: no collective inside a step)"
    elif world > 1 and pst.comm_backend == "fused":
        from litevllm_b200.parallel import fused_ops
        effective_backend = "fused (" + ("two-hop" if fused_ops.decode_allreduce_format(world, torch.bfloat16) == 3
                                        else "one-hop") + " all-reduce in the GEMM epilogue" + \
            (", vocabulary-parallel arg-max" if pst.argmax_ok else ", NCCL logits all-gather") + ")"

    value = B * K / (dev_ms / 1e3)
    e2e_value = B * K / (e2e_ms / 1e3)
    clocks = sampler.summary(*dev_window)
    clocks["under_load_whole_run"] = sampler.summary(min_power_w=250.0)
    result = {
        "metric": METRIC, "value": round(value, 1), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": round(dev_ms / K, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": round(value / PUBLISHED_TPS.get(args.model, BASELINE_TPS), 2), "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": f"{args.model} (random init N(0,0.02))", "global_batch": B, "seq_len": P + 1 + W + K,
                   "prompt_len": P,
                   "parallelism": (f"dp{world} ({world} replicas of the whole engine, {Bl} requests each)"
                                   if mode == "dp" and world > 1 else f"{mode}{world}"),
                   "comm_backend_requested": args.comm_backend, "comm_backend": effective_backend,
                   "self_test": pst.self_test,
                   "l2_policy": "inputs larger than L2 (%.1f GB of weights + KV streamed every step)"
                                % (eng.memory.weight_bytes / 1e9),
                   "tensor_parallel": eng.rc.tensor_parallel_size, "expert_parallel": eng.rc.expert_parallel_size,
                   "kv_cache": str(eng.kv_plan.dtype), "cuda_graph_decode": eng.decode_executor.use_cuda_graph,
                   "reference_note": "the reference admits 16 requests at a time (its stock cap), this engine all 32"},
        "ttft_p50_ms": round(ttft_p50_ms, 2), "ttft_p50_ms_by_submission": [round(t, 2) for t in ttft_runs],
        "ms_per_step_by_ctx": by_ctx,
        "tokens_match_tp1": tokens_match,
        "tokens_check": tokens_check,
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "ms_per_step": round(e2e_ms / K, 4),
                "wall_ms_per_step": round(e2e_wall_ms / K, 4), "wall_value": round(B * K / (e2e_wall_ms / 1e3), 1),
                "h2d_bytes_per_step": h2d_per_step, "d2h_bytes_per_step": d2h_per_step,
                "api": "LiteEngine.add_request + LiteEngine.step (the loop inside LLM.generate)"},
        "gpu_launches": int(dev_replays * per_graph + dev_eager) * world,
        "gpu_launches_detail": {"ranks": world, "graph_replays_per_rank": dev_replays, "kernels_per_graph": per_graph,
                                "eager_native_launches_per_rank": dev_eager},
        "clocks": clocks, "clocks_e2e": sampler.summary(*e2e_window),
        "diag": {"graph_replay_only_ms_per_step": round(graph_only_ms, 4) if graph_only_ms else None,
                 "pdl": os.environ.get("FI_USE_PDL", "1") != "0"},
    }
    if args.profile_json and rank == 0:
        from litevllm_b200.utils.profiling import PROFILER
        Path(args.profile_json).write_text(json.dumps({"result": result, "spans": PROFILER.summary(),
                                                       "engine_stats": eng.stats()}, indent=1, default=str))
    llm.shutdown()
    del llm, eng, pipe
    # ------------------------------------------------------------------ the other BASELINE configurations, short runs
    if world == 1 and args.model == "tinyllama-1.1b" and args.extra_configs:
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        extra = []
        t_extra = time.perf_counter()
        plan = [("dense-9b-awq", [16], 2048, 24), ("gemma4-26b-a4b", [32, 1], 384, 24),
                ("deepseek-mla-moe", [8, 1], 32, 16), ("deepseek-v4-flash", [4, 1], 32, 16)]
        for model, bs, pl, nt in plan:
            if time.perf_counter() - t_extra > args.extra_budget_s:
                extra.append({"model": model, "skipped": f"time budget of {args.extra_budget_s:.0f} s for the extra configurations used up"})
                continue
            try:
                extra += _short_config_runs(args, local_rank, model, bs, pl, nt)
            except Exception as e:   # one broken configuration must not lose the headline line
                extra.append({"model": model, "batches": bs, "prompt_len": pl, "error": repr(e)[:300]})
        result["configs"] = extra
    return result if rank == 0 else {}


def run_reference(args) -> dict:
    from baseline.run_reference import run_reference_bench
    return run_reference_bench(args, METRIC, BASELINE_TPS)


def main():
    args = parse_args()
    res = run_reference(args) if args.impl == "reference" else run_ours(args)
    if res:
        print(json.dumps(res), flush=True)
    if args.impl != "reference" and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        # multi-rank runs end here: the result is printed, and interpreter teardown of process group, graphs and
        # CUDA context in arbitrary order has ended finished ranks with "double free or corruption"
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
