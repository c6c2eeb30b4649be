"""One MoE block with staged experts against the same block with resident experts and against fp32 arithmetic
on the dequantised weights, on the CPU and on the GPU (decode-sized, grouped and tensor-core-sized steps)."""
from types import SimpleNamespace

import pytest
import torch

from litevllm_b200.models.deepseek_mla import RoutedExperts
from litevllm_b200.ops import gguf_quant as gq

E, H, I, K = 16, 512, 256, 4


def _block(device, dtype, weights, budget=None):
    shim = SimpleNamespace(hidden_size=H, extra={"moe_blocks": 1},
                           moe=SimpleNamespace(num_experts=E, expert_intermediate=I, top_k=K))
    ex = RoutedExperts(shim, dtype)
    ex.device = torch.device(device)
    ex.stage_budget = budget
    for which, w in weights.items():
        ex.load(which, w)
    return ex


def _oracle(weights, x, ids, w):
    """fp32 on the Q8_0 round trip of the weights, the activation rounded where the block rounds it."""
    deq = {k: gq.dequantize(gq.quantize_q8_0(v.reshape(-1, v.shape[-1])), 8, v.shape[-1]).view(v.shape) for k, v in weights.items()}
    out = torch.zeros(x.shape[0], H)
    xf = x.float().cpu()
    for t in range(x.shape[0]):
        for k in range(K):
            e = int(ids[t, k])
            a = torch.nn.functional.silu(deq["gate"][e] @ xf[t]) * (deq["up"][e] @ xf[t])
            out[t] += float(w[t, k]) * (deq["down"][e] @ a.to(x.dtype).float())
    return out


def _run(device, dtype):
    g = torch.Generator().manual_seed(5)
    weights = {"gate": torch.randn(E, I, H, generator=g) * 0.05, "up": torch.randn(E, I, H, generator=g) * 0.05,
               "down": torch.randn(E, H, I, generator=g) * 0.05}
    resident = _block(device, dtype, weights)
    per_expert = sum(int(t[0].numel()) * t.element_size() for t in resident.raw.values())
    staged = _block(device, dtype, weights, budget=5 * per_expert + 7)
    worst = 0.0
    for T in (1, 3, 24, 96):                        # 96 x 4 routes over 5 slots: the tensor-core-sized path on a GPU
        x = (torch.randn(T, H, generator=g) * 0.5).to(dtype).to(device)
        ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32).to(device)
        w = torch.rand(T, K, generator=g).to(device)
        got, ref = staged(x, ids, w).float().cpu(), resident(x, ids, w).float().cpu()
        want = _oracle(weights, x, ids.cpu(), w.cpu())
        scale = float(want.norm())
        worst = max(worst, float((got - want).norm()) / scale, float((ref - want).norm()) / scale)
        assert float((got - ref).norm()) / scale < (1e-5 if dtype == torch.float32 else 2e-2), T
    st = staged.stager
    assert st is not None and st.slots == 5 and not staged.raw and st.stats["evictions"] > 0 and st.stats["waves"] > st.stats["steps"]
    return worst


def test_staged_block_on_the_cpu():
    assert _run("cpu", torch.float32) < 1e-3


@pytest.mark.gpu
def test_staged_block_on_the_gpu():
    assert _run("cuda", torch.bfloat16) < 3e-2
