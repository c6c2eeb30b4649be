"""Decode-sized GEMMs as they run inside a decode step: a chain of launches on one stream, every
launch with its own weight matrix (so the weights stream from HBM, not from L2), programmatic
dependent launch on, captured in a CUDA graph.  Prints the device time per launch for each shape of a
model's layer and, with ``--sweep``, for every split-K factor, so the launcher's automatic choice can
be checked against the best fixed one.

    python benchmarks/gemm_chain.py [--tokens 32] [--layers 22] [--sweep] [--tp 1]
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32)
    ap.add_argument("--layers", type=int, default=22)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--inter", type=int, default=5632)
    ap.add_argument("--qkv", type=int, default=2560)
    ap.add_argument("--tp", type=int, default=1, help="shard the shapes as tensor parallelism of this size would")
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--chains", type=int, default=0,
                    help="> 0: run whole layers (qkv, o_proj, gate|up, down in order) as this many independent "
                         "token-slice chains on as many streams inside one graph and print the time per layer")
    ap.add_argument("--trace", action="store_true",
                    help="also print the phase trace of the last launch's first CTA (cycles between marks)")
    args = ap.parse_args()
    import torch

    from litevllm_b200 import ops
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    T, L, H, I, Q, tp = args.tokens, args.layers, args.hidden, args.inter // args.tp, args.qkv // args.tp, args.tp
    bf = torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape, scale=0.02):
        return (torch.randn(*shape, generator=g, device=dev) * scale).to(bf)

    shapes = {"qkv(+rmsnorm)": ("plain_norm", Q, H), "o_proj(+residual)": ("residual", H, H // tp),
              "gate|up(+rmsnorm, silu*up)": ("gated_norm", I, H), "down(+residual)": ("residual", H, I)}
    if args.chains > 0:
        C = args.chains
        Tc = T // C
        layers = []
        for _ in range(L):
            layers.append({n: rnd((2 * N) if k.startswith("gated") else N, K) for n, (k, N, K) in shapes.items()})
        xs = [{n: rnd(Tc, K, scale=0.5) for n, (k, N, K) in shapes.items()} for _ in range(C)]
        rs = [{n: rnd(Tc, N, scale=0.5) for n, (k, N, K) in shapes.items()} for _ in range(C)]
        os_ = [{n: torch.empty(Tc, N, dtype=bf, device=dev) for n, (k, N, K) in shapes.items()} for _ in range(C)]
        streams = [torch.cuda.Stream() for _ in range(C)]

        def chain(c):
            for lw in layers:
                for n, (kind, N, K) in shapes.items():
                    if kind == "plain_norm":
                        ops.linear(xs[c][n], lw[n], out=os_[c][n], rms_eps=1e-5)
                    elif kind == "residual":
                        ops.linear(xs[c][n], lw[n], residual=rs[c][n], out=os_[c][n])
                    else:
                        ops.gated_linear(xs[c][n], lw[n], "silu", out=os_[c][n], rms_eps=1e-5)

        def all_chains():
            cur = torch.cuda.current_stream()
            for c, st in enumerate(streams):
                st.wait_stream(cur)
                with torch.cuda.stream(st):
                    chain(c)
            for st in streams:
                cur.wait_stream(st)

        all_chains()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            all_chains()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ops.check_status(dev)
        us = e0.elapsed_time(e1) * 1e3 / (args.reps * L)
        wbytes = sum(w.numel() * 2 for w in layers[0].values())
        print(json.dumps({"chains": C, "tokens_per_chain": Tc, "layers": L, "us_per_layer_all_chains": round(us, 2),
                          "weights_mb_per_layer": round(wbytes / 1e6, 1),
                          "roofline_us_weights_once": round(wbytes / 6536e3, 2)}))
        return
    results = {}
    for name, (kind, N, K) in shapes.items():
        ws = [rnd((2 * N) if kind.startswith("gated") else N, K) for _ in range(L)]
        x = rnd(T, K, scale=0.5)
        res = rnd(T, N, scale=0.5)
        out = torch.empty(T, N, dtype=bf, device=dev)
        nbytes = ws[0].numel() * 2 + (T * K + T * N) * 2

        def run(splits):
            for w in ws:
                if kind == "plain_norm":
                    ops.linear(x, w, out=out, rms_eps=1e-5, splits=splits)
                elif kind == "residual":
                    ops.linear(x, w, residual=res, out=out, splits=splits)
                else:
                    ops.gated_linear(x, w, "silu", out=out, rms_eps=1e-5, splits=splits)

        row = {}
        for splits in ([0] + list(range(1, 9)) if args.sweep else [0]):
            try:
                run(splits)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    run(splits)
                graph.replay()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(args.reps):
                    graph.replay()
                e1.record()
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / (args.reps * L)
                row["auto" if splits == 0 else f"s{splits}"] = round(us, 2)
            except Exception as e:
                row[f"s{splits}"] = f"error {e!r}"[:60]
        if args.trace:
            from litevllm_b200.ops import _lib
            tr = torch.zeros(8, dtype=torch.int64, device=dev)
            _lib.kernels().fi_dense_gemm_set_trace(tr.data_ptr())
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                run(0)
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            _lib.kernels().fi_dense_gemm_set_trace(None)
            t = tr.tolist()
            names = ["entry", "setup", "pred_done", "accum_ready", "staged", "cluster_met", "stored", "exit"]
            row["trace_us_since_entry"] = {n: round((v - t[0]) / 1965.0, 2) for n, v in zip(names, t) if v}
        ops.check_status(dev)
        results[name] = {"N": N, "K": K, "T": T, "weight_mb": round(ws[0].numel() * 2 / 1e6, 1),
                         "roofline_us_at_6536GBs": round(nbytes / 6536e3, 2), "us_per_launch": row}
        print(name, json.dumps(results[name]), flush=True)
        del ws


if __name__ == "__main__":
    main()
