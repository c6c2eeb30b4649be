"""Device-timed micro-benchmark of the fused compute+collective GEMMs against the GEMM + NCCL
baseline, with a roofline fraction per shape.

Launch one process per GPU:
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29533 benchmarks/fused_collectives.py [--iters 20] [--out FILE.json]

For every (op, T, N, K) the op is captured ``iters`` times in one CUDA graph, the graph is replayed
after warm-up between CUDA events, and the per-call time is the max over ranks.  Roofline per call:
the slower of FLOPs / measured bf16 GEMM peak, bytes that must cross NVLink per GPU / 770 GB/s, and
(for decode shapes, where the weights stream from HBM once) weight bytes / measured HBM bandwidth.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

NVLINK_GBS = 770.0


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d.get("hbm_gbs", 6650.0)), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--replays", type=int, default=5)
    ap.add_argument("--out", default=None)
    ap.add_argument("--prefill-tokens", type=int, default=4096)
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    from litevllm_b200 import ops
    from litevllm_b200.parallel import fused_ops, state as pstate
    from litevllm_b200.parallel.symm import SymmetricHeap

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world < 2:
        raise SystemExit("run under torchrun with at least 2 ranks")
    st = pstate.init_parallel(tp=world, comm_backend="fused")
    rank = st.rank
    dev = torch.device("cuda", st.local_rank)
    st.symm = SymmetricHeap(rank, world, dev, recv_bytes=1 << 30, xbuf_bytes=128 << 20)
    hbm, tflops, src = peaks()

    class Layer:
        quant_method = None
        bias = None

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(iters):
                fn()
        g.replay()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.replays):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / (iters * args.replays)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        del g
        return float(t.item())          # microseconds per call

    Tp = args.prefill_tokens // world * world
    shapes = [  # (label, T, N, K_total)
        ("tinyllama o_proj decode", 32, 2048, 2048), ("tinyllama down decode", 32, 2048, 5632 // world * world),
        ("9b o_proj decode", 16, 4096, 4096), ("9b down decode", 16, 4096, 12288),
        ("tinyllama down prefill", Tp, 2048, 5632 // world * world), ("9b down prefill", Tp, 4096, 12288),
    ]
    rows = []
    gen = torch.Generator(device=dev).manual_seed(7 + rank)
    for label, T, N, Kt in shapes:
        K = Kt // world
        K = K // 64 * 64
        x = (torch.randn(T, K, generator=gen, device=dev) * 0.5).bfloat16()
        w = (torch.randn(N, K, generator=gen, device=dev) * 0.05).bfloat16()
        res = torch.zeros(T, N, device=dev, dtype=torch.bfloat16)
        out = torch.empty(T, N, device=dev, dtype=torch.bfloat16)
        layer = Layer()
        layer.weight, layer.out_features = w, N
        # decode shapes use an inline-epoch low-latency format: one hop (every rank sends its partial to
        # every peer) or, from four ranks on, two hops (partials to the owner of a column chunk, 16-bit
        # sums broadcast back); both are timed, "fused_us" is the one the engine picks for this world size
        decode = T <= 256
        xfer16 = 1 if not decode else fused_ops.decode_allreduce_format(world, torch.bfloat16)
        elem = 2 if not decode else 8
        iters = args.iters if T <= 256 else 4
        flops = 2.0 * T * N * K
        t_compute = flops / (tflops * 1e12) * 1e6
        t_hbm = (N * K * 2 + T * K * 2 + T * N * 2) / (hbm * 1e9) * 1e6

        def fused_ar():
            fused_ops._fused_gemm_allreduce(layer, x, res, out, st.symm, xfer16)

        def nccl_ar():
            y = ops.linear(x, w)
            dist.all_reduce(y)
            torch.add(y, res, out=out)

        def local_only():
            ops.linear(x, w, out=out)

        t_local = timed(local_only, iters)
        t_f, t_n = timed(fused_ar, iters), timed(nccl_ar, iters)
        per_format = {}
        if decode:
            for name, fmt in (("one_hop_us", 2), ("two_hop_us", 3)):
                per_format[name] = round(timed(lambda: fused_ops._fused_gemm_allreduce(layer, x, res, out, st.symm, fmt),
                                               iters), 2)
        if decode and xfer16 == 3:
            # per GPU: (world - 1) / world of the tile out as fp32 words with their epochs, the same share back as 16-bit sums
            link = (world - 1) / world * T * N * (8 + 4) / (NVLINK_GBS * 1e9) * 1e6
        else:
            link = (world - 1) * T * N * elem / (NVLINK_GBS * 1e9) * 1e6
        roof = max(t_compute, link, t_hbm)
        rows.append({"op": "gemm+all_reduce", "shape": label, "T": T, "N": N, "K_per_rank": K, "fused_us": round(t_f, 2),
                     "nccl_us": round(t_n, 2), "local_gemm_us": round(t_local, 2), "roofline_us": round(roof, 2),
                     "bound": "compute" if roof == t_compute else ("nvlink" if roof == link else "hbm"),
                     "frac_of_roofline": round(roof / t_f, 3), "speedup_vs_nccl": round(t_n / t_f, 2), **per_format})
        if T >= world * 128:
            rpr = T // world
            res_s = torch.zeros(rpr, N, device=dev, dtype=torch.bfloat16)
            out_s = torch.empty(rpr, N, device=dev, dtype=torch.bfloat16)

            def fused_rs():
                fused_ops.gemm_reduce_scatter(x, w, res_s, rpr, out_s, True)

            def nccl_rs():
                y = ops.linear(x, w)
                dist.reduce_scatter_tensor(out_s, y)
                out_s.add_(res_s)

            t_f, t_n = timed(fused_rs, iters), timed(nccl_rs, iters)
            link = (world - 1) * rpr * N * 2 / (NVLINK_GBS * 1e9) * 1e6
            roof = max(t_compute, link)
            rows.append({"op": "gemm+reduce_scatter", "shape": label, "T": T, "N": N, "K_per_rank": K,
                         "fused_us": round(t_f, 2), "nccl_us": round(t_n, 2), "roofline_us": round(roof, 2),
                         "bound": "compute" if roof == t_compute else "nvlink",
                         "frac_of_roofline": round(roof / t_f, 3), "speedup_vs_nccl": round(t_n / t_f, 2)})
            # all-gather -> GEMM: column-parallel weight [N/world, K_total], tokens sharded by rows
            Kag = Kt // 64 * 64 if Kt <= 4096 else 4096
            Nag = (N // world) // 128 * 128
            xs = (torch.randn(rpr, Kag, generator=gen, device=dev) * 0.5).bfloat16()
            wc = (torch.randn(Nag, Kag, generator=gen, device=dev) * 0.05).bfloat16()
            out_ag = torch.empty(T, Nag, device=dev, dtype=torch.bfloat16)
            full = torch.empty(T, Kag, device=dev, dtype=torch.bfloat16)

            def fused_ag():
                fused_ops.allgather_gemm(xs, wc, T, rpr, out_ag)

            def nccl_ag():
                dist.all_gather_into_tensor(full, xs)
                ops.linear(full, wc, out=out_ag)

            t_f, t_n = timed(fused_ag, iters), timed(nccl_ag, iters)
            fl = 2.0 * T * Nag * Kag / (tflops * 1e12) * 1e6
            link = (world - 1) * rpr * Kag * 2 / (NVLINK_GBS * 1e9) * 1e6
            roof = max(fl, link)
            rows.append({"op": "all_gather+gemm", "shape": label, "T": T, "N": Nag, "K_per_rank": Kag,
                         "fused_us": round(t_f, 2), "nccl_us": round(t_n, 2), "roofline_us": round(roof, 2),
                         "bound": "compute" if roof == fl else "nvlink",
                         "frac_of_roofline": round(roof / t_f, 3), "speedup_vs_nccl": round(t_n / t_f, 2)})
    ops.check_status(dev)
    if rank == 0:
        result = {"world": world, "peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "nvlink_gbs": NVLINK_GBS, "source": src},
                  "rows": rows}
        print(json.dumps(result, indent=1), flush=True)
        if args.out:
            Path(args.out).write_text(json.dumps(result, indent=1))
    torch.cuda.synchronize()
    dist.barrier()
    pstate.destroy_parallel(destroy_group=False)
    os._exit(0)


if __name__ == "__main__":
    main()
