"""The allocation-free decode entry point, called through its exported C symbol.

Some users of the kernel library cannot hand it scratch buffers: a C/C++ program that links the
shared object without any tensor allocator, or a server that gave its whole device-memory budget to
the KV pool when it started.  ``fi_paged_decode_noalloc`` keeps the split-KV partials in a fixed
array inside the library instead.  This test checks it against the regular entry point on two calls
in a row (the second call sees the first call's leftovers in the shared array) and checks that an
oversized request is refused.  It lives in a file that sorts last so that a ``-x`` run has already
exercised everything else when it gets here; it does not depend on any earlier test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, q, kc, vc, out, bt, sl, nh, nkv, hd, scale, splits, window=0, softcap=0.0):
    fn = lib.fi_paged_decode_noalloc
    B = sl.shape[0]
    return fn(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), bt.data_ptr(),
              sl.data_ptr(), B, nh, nkv, hd, bt.shape[1], kc.shape[2], window, scale, softcap, 0, 1.0, 1.0,
              splits, 0, torch.cuda.current_stream().cuda_stream)


def test_noalloc_decode_matches_regular_entry_point():
    from litevllm_b200 import ops
    from litevllm_b200.ops import _lib, reference
    lib = _lib.kernels()
    assert isinstance(lib, ctypes.CDLL) and hasattr(lib, "fi_paged_decode_noalloc")
    dev = "cuda"
    torch.manual_seed(11)
    nh, nkv, hd, bs = 32, 4, 64, 16
    scale = 1.0 / math.sqrt(hd)
    for round_idx, (lens, splits) in enumerate([([300, 17, 1, 129, 64, 250], 4), ([90, 511, 33], 3)]):
        B = len(lens)
        max_blocks = (max(lens) + bs - 1) // bs + 1
        nb = 1 + B * max_blocks
        kc = (torch.randn(nb, nkv, bs, hd, device=dev) * 0.7).bfloat16()
        vc = (torch.randn(nb, nkv, bs, hd, device=dev) * 0.7).bfloat16()
        bt = torch.zeros(B, max_blocks, dtype=torch.int32, device=dev)
        perm = torch.randperm(nb - 1, device=dev) + 1
        used = 0
        for b in range(B):
            n = (lens[b] + bs - 1) // bs
            bt[b, :n] = perm[used:used + n].to(torch.int32)
            used += n
        q = torch.randn(B, nh * hd, device=dev).bfloat16()
        sl = torch.tensor(lens, dtype=torch.int32, device=dev)
        want = ops.paged_attention_decode(q, kc, vc, bt, sl, nh, nkv, hd, scale, splits=splits,
                                          max_kv_len=max(lens))
        got = torch.full_like(want, float("nan"))
        rc = _call_noalloc(lib, q, kc, vc, got, bt, sl, nh, nkv, hd, scale, splits)
        assert rc == 0, f"round {round_idx}: return code {rc}"
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs()
        tol = 2e-2 + 2e-2 * want.float().abs()
        assert bool((err <= tol).all()), f"round {round_idx}: max abs err {float(err.max())}"
        # second oracle: the plain PyTorch fp32 attention over the same paged cache (the regular entry
        # point runs the same kernel, so agreeing with it alone would not catch a shared mistake)
        cu = torch.arange(B + 1, dtype=torch.int32)
        oracle = reference.paged_attention(q.cpu(), kc.cpu(), vc.cpu(), bt.cpu(), sl.cpu(), cu, nh, nkv, hd, scale,
                                           0, 0.0, 1.0, 1.0).float()
        err = (got.float().cpu() - oracle).abs()
        assert bool((err <= 2e-2 + 2e-2 * oracle.abs()).all()), f"round {round_idx}: vs fp32 oracle {float(err.max())}"


def test_noalloc_decode_rejects_oversized_request():
    from litevllm_b200.ops import _lib
    lib = _lib.kernels()
    dev = "cuda"
    # 4096 * 64 * 8 * (128 + 2) floats is far beyond the 2 Mi-float array: must be refused unlaunched
    B, nh, nkv, hd, splits = 4096, 64, 8, 128, 8
    dummy = torch.zeros(16, device=dev)
    sl = torch.zeros(B, dtype=torch.int32, device=dev)
    bt = torch.zeros(B, 1, dtype=torch.int32, device=dev)
    kc = torch.zeros(1, nkv, 16, hd, device=dev, dtype=torch.bfloat16)
    rc = lib.fi_paged_decode_noalloc(dummy.data_ptr(), nh * hd, kc.data_ptr(), kc.data_ptr(), dummy.data_ptr(),
                                     bt.data_ptr(), sl.data_ptr(), B, nh, nkv, hd, 1, 16, 0, 0.1, 0.0, 0, 1.0, 1.0,
                                     splits, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == -20
    torch.cuda.synchronize()


def test_noalloc_decode_single_split_has_no_size_limit():
    """With one split the kernel writes straight to the output and uses no scratch, so a batch whose
    B * nh * (hd + 2) exceeds the built-in array is still served (short contexts keep it cheap)."""
    from litevllm_b200 import ops
    from litevllm_b200.ops import _lib
    lib = _lib.kernels()
    dev = "cuda"
    torch.manual_seed(5)
    B, nh, nkv, hd, bs = 600, 32, 4, 128, 16
    assert B * nh * (hd + 2) > 2 * 1024 * 1024
    scale = 1.0 / math.sqrt(hd)
    lens = [1 + (i * 7) % 40 for i in range(B)]
    max_blocks = 3
    nb = 1 + B * max_blocks
    kc = (torch.randn(nb, nkv, bs, hd, device=dev) * 0.5).bfloat16()
    vc = (torch.randn(nb, nkv, bs, hd, device=dev) * 0.5).bfloat16()
    bt = (1 + torch.arange(B * max_blocks, device=dev, dtype=torch.int32)).view(B, max_blocks).contiguous()
    q = torch.randn(B, nh * hd, device=dev).bfloat16()
    sl = torch.tensor(lens, dtype=torch.int32, device=dev)
    want = ops.paged_attention_decode(q, kc, vc, bt, sl, nh, nkv, hd, scale, splits=1, max_kv_len=max(lens))
    got = torch.full_like(want, float("nan"))
    rc = _call_noalloc(lib, q, kc, vc, got, bt, sl, nh, nkv, hd, scale, 1)
    assert rc == 0
    torch.cuda.synchronize()
    assert bool(((got.float() - want.float()).abs() <= 2e-2 + 2e-2 * want.float().abs()).all())
    # bad head counts are an argument error, not a crash on the host
    assert lib.fi_paged_decode_noalloc(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), got.data_ptr(),
                                       bt.data_ptr(), sl.data_ptr(), B, nh, 0, hd, max_blocks, bs, 0, scale, 0.0, 0,
                                       1.0, 1.0, 2, 0, torch.cuda.current_stream().cuda_stream) == -10
