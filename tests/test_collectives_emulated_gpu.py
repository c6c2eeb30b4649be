"""The push / poll / ownership code of the fused compute+collective kernels on ONE GPU.

``SymmetricHeap.emulated(world, device)`` lays the heaps of ``world`` ranks side by side in one
allocation; every "rank" is a launch with its own rank number, operands and heap view, and its peer
pointers address the neighbouring regions.  Launches on one GPU cannot wait for one another, so a
fused call is driven phase by phase: the push phase of every rank, then the reduce phase of every
rank, then (two-hop all-reduce) the collect phase.  What runs is the same device code a multi-GPU job
runs (peer stores with inline epochs, flag release/acquire, owner reduction, epoch bookkeeping); only
the transport (local memory instead of NVLink) differs.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

PUSH, REDUCE, COLLECT = 1, 2, 4


class _Layer:
    quant_method, bias = None, None


def _close(got, want, tol, what):
    err = (got.float() - want.float()).abs()
    assert bool((err <= tol + tol * want.float().abs()).all()), f"{what}: max abs err {float(err.max())}"


@pytest.fixture(scope="module")
def heaps_by_world():
    from litevllm_b200.parallel.symm import SymmetricHeap
    dev = torch.device("cuda", 0)
    made = {}

    def get(world):
        if world not in made:
            made[world] = SymmetricHeap.emulated(world, dev)
        return made[world]
    yield get
    torch.cuda.synchronize()
    for hs in made.values():
        for h in hs:
            h.close()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("fmt", [2, 3, 0])
def test_gemm_allreduce_emulated_ranks(heaps_by_world, world, fmt):
    """GEMM -> all-reduce (+ bias on rank 0, + residual) for the one-hop inline-epoch form (2), the
    two-hop form (3) and the flagged fp32 form (0): every rank must end with the fp32 oracle."""
    from litevllm_b200 import ops
    from litevllm_b200.parallel import fused_ops
    dev = torch.device("cuda", 0)
    heaps = heaps_by_world(world)
    phase_list = [PUSH, REDUCE, COLLECT] if fmt == 3 else [PUSH, REDUCE]
    for T, N, K in [(32, 512, 256), (7, 384, 320), (64, 2048, 128), (200, 256, 64)]:
        g = torch.Generator(device=dev).manual_seed(T * 31 + N + world)
        xs = [(torch.randn(T, K, generator=g, device=dev) * 0.5).bfloat16() for _ in range(world)]
        ws = [(torch.randn(N, K, generator=g, device=dev) * 0.05).bfloat16() for _ in range(world)]
        bias = (torch.randn(N, generator=g, device=dev) * 0.1).bfloat16()
        res = torch.randn(T, N, generator=g, device=dev).bfloat16()
        want = sum(x.float() @ w.float().t() for x, w in zip(xs, ws)) + bias.float() + res.float()
        for rep in range(2):                                  # both slab parities
            outs = [torch.full((T, N), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(world)]
            for ph in phase_list:
                for r in range(world):
                    layer = _Layer()
                    layer.weight, layer.out_features, layer.bias = ws[r], N, bias
                    fused_ops._fused_gemm_allreduce(layer, xs[r], res, outs[r], heaps[r], fmt, phases=ph)
            torch.cuda.synchronize()
            ops.check_status(dev)
            for r in range(world):
                _close(outs[r], want, 4e-2, f"world {world} fmt {fmt} T{T} N{N} rep {rep} rank {r}")
            for r in range(1, world):                         # bitwise identical on every rank
                assert torch.equal(outs[0], outs[r]), f"rank {r} differs from rank 0 (fmt {fmt})"
    assert all(h.epoch_value() > 0 for h in heaps)
    assert len({h.epoch_value() for h in heaps}) == 1


@pytest.mark.parametrize("world", [2, 4])
def test_gemm_reduce_scatter_emulated_ranks(heaps_by_world, world):
    from litevllm_b200 import ops
    from litevllm_b200.parallel import fused_ops
    dev = torch.device("cuda", 0)
    heaps = heaps_by_world(world)
    rpr, N, K = 128, 384, 256
    T = rpr * world
    g = torch.Generator(device=dev).manual_seed(77 + world)
    xs = [(torch.randn(T, K, generator=g, device=dev) * 0.5).bfloat16() for _ in range(world)]
    ws = [(torch.randn(N, K, generator=g, device=dev) * 0.05).bfloat16() for _ in range(world)]
    res = [torch.randn(rpr, N, generator=g, device=dev).bfloat16() for _ in range(world)]
    full = sum(x.float() @ w.float().t() for x, w in zip(xs, ws))
    for rep in range(2):
        outs = [torch.full((rpr, N), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(world)]
        for ph in (PUSH, REDUCE):
            for r in range(world):
                fused_ops.gemm_reduce_scatter(xs[r], ws[r], res[r], rpr, out_shard=outs[r], heap=heaps[r], phases=ph)
        torch.cuda.synchronize()
        ops.check_status(dev)
        for r in range(world):
            _close(outs[r], full[r * rpr:(r + 1) * rpr] + res[r].float(), 5e-2, f"reduce-scatter world {world} rank {r}")


@pytest.mark.parametrize("world", [2, 8])
def test_argmax_vocab_parallel_emulated_ranks(heaps_by_world, world):
    from litevllm_b200 import ops
    from litevllm_b200.parallel import fused_ops
    dev = torch.device("cuda", 0)
    heaps = heaps_by_world(world)
    rows, V = 33, 4000
    g = torch.Generator(device=dev).manual_seed(5)
    full = torch.randn(rows, V * world, generator=g, device=dev)
    full[3, 17] = full[3, V + 5] = 50.0            # a tie across ranks: the lowest global index wins
    full[4, V * (world - 1) + 9] = 60.0
    want = full.argmax(-1)
    want[3] = 17
    parts = [full[:, r * V:(r + 1) * V].contiguous() for r in range(world)]
    for rep in range(2):
        outs = [torch.full((rows,), -1, device=dev, dtype=torch.int64) for _ in range(world)]
        for ph in (PUSH, REDUCE):
            for r in range(world):
                fused_ops.argmax_vocab_parallel(parts[r], r * V, out=outs[r], heap=heaps[r], phases=ph)
        torch.cuda.synchronize()
        ops.check_status(dev)
        for r in range(world):
            assert torch.equal(outs[r], want), f"rank {r} rep {rep}"


def test_moe_combine_allreduce_emulated_ranks(heaps_by_world):
    from litevllm_b200 import ops
    from litevllm_b200.ops import _lib
    dev = torch.device("cuda", 0)
    world = 2
    heaps = heaps_by_world(world)
    T, K, H = 24, 4, 512
    g = torch.Generator(device=dev).manual_seed(400)
    ys = [torch.randn(T * K, H, generator=g, device=dev).bfloat16() for _ in range(world)]
    wts = torch.rand(T, K, generator=g, device=dev)
    res = torch.randn(T, H, generator=g, device=dev).bfloat16()
    want = sum((y.float().view(T, K, H) * wts[:, :, None]).sum(1) for y in ys) + res.float()
    for rep in range(2):
        outs = [torch.full((T, H), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(world)]
        for ph in (PUSH, REDUCE):
            for r in range(world):
                comm = heaps[r].comm_desc(mode=1, T=T, N=H, xfer_16bit=2, phases=ph)
                rc = _lib.kernels().fi_moe_combine_allreduce(ops._p(ys[r]), None, ops._p(wts), ops._p(res), ops._p(outs[r]),
                                                             T, K, H, 0, ops._p(ops.status_word(dev)), ops._stream(),
                                                             ctypes.byref(comm))
                assert rc == 0
        torch.cuda.synchronize()
        ops.check_status(dev)
        for r in range(world):
            _close(outs[r], want, 4e-2, f"moe combine rank {r} rep {rep}")
