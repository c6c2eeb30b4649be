"""Small, self-contained launches of each hot kernel: device-timed with CUDA events, and sized so that
a profiler capture of one or two launches ends by itself (inputs larger than the 126 MB L2 where
DRAM figures matter, at most a few GB on the device).

    python benchmarks/kernel_cases.py --case dense_gemm_decode [--iters 20] [--json out.json]
    python benchmarks/kernel_cases.py --list

Each case prints achieved bandwidth / FLOP rate next to the measured peaks in MEASURED_PEAKS.json
(fallback 6650 GB/s, 1590 TFLOP/s).  For a profile:
    ncu --set full --clock-control none -k regex:<kernel> -s 4 -c 2 -o prof python benchmarks/kernel_cases.py --case <case> --iters 4
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d.get("hbm_gbs", 6650.0)), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="dense_gemm_decode")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", default=None)
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--kv-block", type=int, default=16, help="tokens per KV page in the prefill attention cases")
    args = ap.parse_args()

    import torch

    from litevllm_b200 import ops
    from litevllm_b200.ops import awq, gguf_quant as gq, moe

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(0)
    bf = torch.bfloat16

    def rnd(*shape, scale=1.0, dtype=bf):
        return (torch.randn(*shape, generator=g, device=dev) * scale).to(dtype)

    cases = {}

    def case(name):
        def deco(fn):
            cases[name] = fn
            return fn
        return deco

    # every case returns (callable, algorithmic bytes per call, flops per call, note)
    @case("dense_gemm_decode")
    def _():
        T, N, K = 32, 16384, 8192                       # 268 MB of weights: streams from HBM
        x, w = rnd(T, K), rnd(N, K, scale=0.02)
        out = torch.empty(T, N, dtype=bf, device=dev)
        return (lambda: ops.linear(x, w, out=out)), (N * K + T * K + T * N) * 2, 2.0 * T * N * K, f"T={T} N={N} K={K} bf16"

    @case("dense_gemm_rmsnorm_decode")
    def _():
        T, N, K = 32, 16384, 8192
        x, w = rnd(T, K), rnd(N, K, scale=0.02)
        out = torch.empty(T, N, dtype=bf, device=dev)
        return (lambda: ops.linear(x, w, out=out, rms_eps=1e-5)), (N * K + T * K + T * N) * 2, 2.0 * T * N * K, \
            f"T={T} N={N} K={K} bf16, RMSNorm of the token rows inside the kernel"

    @case("dense_gemm_gated_decode")
    def _():
        T, I, K = 32, 8192, 8192
        x, w = rnd(T, K), rnd(2 * I, K, scale=0.02)
        out = torch.empty(T, I, dtype=bf, device=dev)
        return (lambda: ops.gated_linear(x, w, "silu", out=out)), (2 * I * K + T * K + T * I) * 2, 4.0 * T * I * K, \
            f"T={T} I={I} K={K} gate|up with SiLU*up epilogue"

    @case("dense_gemm_prefill")
    def _():
        T, N, K = 8192, 8192, 8192
        x, w = rnd(T, K), rnd(N, K, scale=0.02)
        out = torch.empty(T, N, dtype=bf, device=dev)
        return (lambda: ops.linear(x, w, out=out)), (N * K + T * K + T * N) * 2, 2.0 * T * N * K, f"T={T} N={N} K={K} bf16"

    @case("int4_gemm_decode")
    def _():
        T, N, K, G = 16, 32768, 8192, 128                # 134 MB of packed nibbles
        nib = torch.randint(0, 16, (N, K), generator=g, device=dev, dtype=torch.uint8)
        sc = (torch.rand(N, K // G, generator=g, device=dev) * 0.01 + 0.001).to(torch.float16)
        zp = torch.randint(0, 16, (N, K // G), generator=g, device=dev, dtype=torch.uint8)
        w = awq.Int4Weight(nib, sc, zp, G, torch.float16)
        x = rnd(T, K, dtype=torch.float16)
        out = torch.empty(T, N, dtype=torch.float16, device=dev)
        return (lambda: awq.int4_linear(x, w, out=out)), N * K // 2 + N * (K // G) * 3 + (T * K + T * N) * 2, \
            2.0 * T * N * K, f"T={T} N={N} K={K} AWQ group {G} with zero points"

    @case("decode_attention")
    def _():
        B, ctx, nh, nkv, hd, bs = 64, 4096, 32, 8, 128, 16
        blocks_per = ctx // bs
        nb = B * blocks_per + 1
        kc, vc = rnd(nb, nkv, bs, hd), rnd(nb, nkv, bs, hd)          # 2 x 537 MB
        bt = (torch.arange(B * blocks_per, device=dev, dtype=torch.int32) + 1).view(B, blocks_per)
        sl = torch.full((B,), ctx, dtype=torch.int32, device=dev)
        qkv = rnd(B, (nh + 2 * nkv) * hd)
        return (lambda: ops.paged_attention_decode(qkv, kc, vc, bt, sl, nh, nkv, hd, hd ** -0.5, 0, 0.0, 1.0, 1.0,
                                                   max_kv_len=ctx)), \
            2 * B * ctx * nkv * hd * 2, 4.0 * B * nh * ctx * hd, f"B={B} ctx={ctx} {nh}q/{nkv}kv hd={hd} block {bs}"

    @case("prefill_attention")
    def _():
        B, L, nh, nkv, hd, bs = 8, 2048, 32, 8, 128, args.kv_block
        blocks_per = L // bs
        nb = B * blocks_per + 1
        kc, vc = rnd(nb, nkv, bs, hd), rnd(nb, nkv, bs, hd)
        bt = (torch.arange(B * blocks_per, device=dev, dtype=torch.int32) + 1).view(B, blocks_per)
        sl = torch.full((B,), L, dtype=torch.int32, device=dev)
        cu = (torch.arange(B + 1, device=dev, dtype=torch.int32) * L)
        qkv = rnd(B * L, (nh + 2 * nkv) * hd)
        return (lambda: ops.paged_attention_prefill(qkv, kc, vc, bt, sl, cu, L, nh, nkv, hd, hd ** -0.5)), \
            (B * L * (nh + 2 * nkv) * hd + B * L * nh * hd) * 2, 4.0 * B * nh * L * L * hd / 2, \
            f"B={B} L={L} causal {nh}q/{nkv}kv hd={hd} page {bs}"

    @case("prefill_attention_hd64")
    def _():
        B, L, nh, nkv, hd, bs = 8, 1024, 32, 4, 64, args.kv_block     # one TinyLlama prefill micro-batch
        blocks_per = L // bs
        nb = B * blocks_per + 1
        kc, vc = rnd(nb, nkv, bs, hd), rnd(nb, nkv, bs, hd)
        bt = (torch.arange(B * blocks_per, device=dev, dtype=torch.int32) + 1).view(B, blocks_per)
        sl = torch.full((B,), L, dtype=torch.int32, device=dev)
        cu = (torch.arange(B + 1, device=dev, dtype=torch.int32) * L)
        qkv = rnd(B * L, (nh + 2 * nkv) * hd)
        return (lambda: ops.paged_attention_prefill(qkv, kc, vc, bt, sl, cu, L, nh, nkv, hd, hd ** -0.5)), \
            (B * L * (nh + 2 * nkv) * hd + B * L * nh * hd) * 2, 4.0 * B * nh * L * L * hd / 2, \
            f"B={B} L={L} causal {nh}q/{nkv}kv hd={hd} page {bs}"

    @case("gguf_moe_decode")
    def _():
        # routed experts of one DeepSeek-shaped layer at decode size: 8 tokens x top-6 over 256 experts,
        # IQ2_XXS gate / up, Q2_K down (1.8 GB of expert blocks on the device; ~48 experts are touched per call)
        import litevllm_b200.models.deepseek_mla as dm
        from litevllm_b200.models.arch import arch_from_hf_config
        from litevllm_b200.models.presets import get_preset
        arch = arch_from_hf_config(get_preset("deepseek-mla-moe"))
        E, I, H, K = arch.moe.num_experts, arch.moe.expert_intermediate, arch.hidden_size, arch.moe.top_k
        with torch.device(dev):
            ex = dm.RoutedExperts(arch, bf)
        ex.device = dev
        for which, ty, rows, cols, seed in (("gate", 16, I, H, 1), ("up", 16, I, H, 2), ("down", 10, H, I, 3)):
            raw = gq.random_blocks(ty, 8 * rows, cols, seed=seed, scale=0.05).to(dev)
            raw = raw.repeat(E // 8, 1).view(E, rows, -1).contiguous()          # 8 distinct experts, tiled to 256
            ex.raw[which], ex.types[which] = raw, ty
        T = 8
        x = rnd(T, H)
        ids = torch.stack([torch.randperm(E, generator=g, device=dev)[:K] for _ in range(T)]).to(torch.int32)
        w = torch.rand(T, K, generator=g, device=dev)
        nbytes = T * K * (2 * I * H * 66 // 256 + H * I * 84 // 256)
        return (lambda: ex(x, ids, w)), nbytes, 2.0 * T * K * 3 * I * H, \
            f"T={T} top-{K} of {E} experts, H={H} I={I}, IQ2_XXS gate/up + Q2_K down, int8 activations (align + 2 kernels + combine)"

    @case("rmsnorm")
    def _():
        T, H = 65536, 4096                                # 537 MB in + out
        x, w = rnd(T, H), rnd(H)
        out = torch.empty_like(x)
        return (lambda: ops.rmsnorm(x, w, 1e-5, out=out)), 2 * T * H * 2, 0.0, f"T={T} H={H}"

    @case("gguf_q8_0_gemv")
    def _():
        M, N, K = 4, 32768, 8192
        ty = gq.GGML_TYPES["Q8_0"]
        raw = gq.random_blocks(ty, N, K, seed=1, scale=0.02, device=dev)
        x = rnd(M, K)
        out = torch.empty(M, N, dtype=torch.float32, device=dev)
        return (lambda: gq.gguf_linear(x, raw, ty, K, out=out, out_dtype=torch.float32)), raw.numel(), 2.0 * M * N * K, \
            f"M={M} N={N} K={K} Q8_0 blocks ({raw.numel() / 1e6:.0f} MB)"

    @case("moe_int4_decode")
    def _():
        T, E, K_top, H, I, G = 32, 128, 8, 2816, 704, 32
        def make(rows, cols):
            nib = torch.randint(0, 16, (E * rows, cols), generator=g, device=dev, dtype=torch.uint8)
            sc = (torch.rand(E * rows, cols // G, generator=g, device=dev) * 0.01 + 0.001).to(bf)
            return awq.Int4Weight(nib, sc, None, G, bf)
        wg, wd = make(2 * I, H), make(H, I)
        x = rnd(T, H)
        logits = torch.randn(T, E, generator=g, device=dev)
        ids, wts = moe.route(logits, K_top, "softmax")
        touched = min(E, T * K_top)
        return (lambda: moe.fused_experts(x, wg, wd, ids, wts, E, 0, "gelu_tanh")), \
            touched * (3 * I * H) // 2, 2.0 * T * K_top * 3 * I * H, \
            f"T={T} E={E} top-{K_top} H={H} I={I} int4 group {G} (align + gather + 2 grouped GEMMs + combine)"

    if args.list:
        print("\n".join(cases))
        return
    fn, nbytes, flops, note = cases[args.case]()
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    # L2 flush: READ a buffer larger than the 126 MB L2 (a write would leave dirty lines whose
    # write-back is then charged to the kernel under test)
    flush = torch.zeros(512 << 20, dtype=torch.uint8, device=dev).view(torch.int64)
    times = []
    for _ in range(args.iters):
        flush.sum()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    ops.check_status(dev)
    times.sort()
    us = times[len(times) // 2]
    hbm, tflops, src = peaks()
    res = {"case": args.case, "note": note, "median_us": round(us, 2), "min_us": round(times[0], 2),
           "gbs": round(nbytes / us / 1e3, 1), "frac_of_hbm": round(nbytes / us / 1e3 / hbm, 3),
           "tflops": round(flops / us / 1e6, 1), "frac_of_bf16_peak": round(flops / us / 1e6 / tflops, 3),
           "peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": src}, "l2": "flushed (512 MB read) between iterations"}
    print(json.dumps(res))
    if args.json:
        Path(args.json).write_text(json.dumps(res, indent=1))


if __name__ == "__main__":
    main()
