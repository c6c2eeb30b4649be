"""DeepSeek-V2/V3-style decoder: multi-head latent attention (MLA) + mixture of experts.

Attention: ``q = q_b(norm(q_a(x)))`` (or a direct q projection), ``[latent | k_rope] = kv_a(x)``,
``[k_nope | v] = kv_b(norm(latent))``; rotary on the 64 rope channels of q and of the shared k_rope;
softmax scale ``1/sqrt(nope + rope)``.  This implementation materialises per-head keys/values into
the paged cache (head layout ``[rope | nope | pad]`` so the rotary kernel's "first rot_dim channels"
convention applies; keys and values are padded to a common 256-wide head) and reuses the paged
attention kernels; the latent-absorbed cache form is a later optimisation.
MoE: router ``gate`` with sigmoid (or softmax) scoring, selection bias, top-k, renormalisation and
routed scaling; routed experts stay in their GGUF block formats (IQ2_XXS / Q2_K / Q8_0) and run
through the routed-expert kernels; shared experts and the leading dense layers are ordinary gated
MLPs.  Experts are sharded over expert-parallel ranks, attention over tensor-parallel ranks.
Reference: the reference serves only the V4-Flash variant (vllm/model_executor/models/
deepseek_v4_flash/*); its MoE numerics (sigmoid/softplus scoring, shared expert, clamp) are followed.
"""
from __future__ import annotations

import os

import torch
from torch import nn

from .. import ops
from ..layers.linear import LiteLinear
from ..logger import init_logger
from ..layers.rope import get_cos_sin
from ..ops import gguf_quant as gq
from ..ops import moe as moe_ops
from ..ops import _lib, _p, _stream, _count, scratch
from ..parallel import state as pstate
from ..utils.profiling import stage
from .arch import ModelArch
from .llama import RMSNormWeight

logger = init_logger(__name__)

# Routed experts from GGUF blocks: "auto" sorts the routes by expert and runs the grouped kernels when a
# step has at least as many routes as local experts, "on" / "off" force one form.
_GROUPED = os.environ.get("FI_GGUF_MOE_GROUPED", "auto")
# Q2_K / IQ2_XXS experts: quantise the activations to int8 (a scale per 32 values) and use integer dot products
# (FI_GGUF_MOE_Q8=0 keeps 16-bit activations and float arithmetic).
_Q8 = os.environ.get("FI_GGUF_MOE_Q8", "1") != "0"
# Multi-head latent attention in absorbed form (one 576-value cache row per token instead of per-head K and V):
# on when the kv_b projections are dense 16-bit matrices on a GPU; FI_MLA_ABSORBED=0 keeps the materialised form.
_ABSORBED = os.environ.get("FI_MLA_ABSORBED", "1") != "0"
_MATERIALISED_MAX_TOKENS = 8192
# Routed experts: from this many routes per local expert (on average) a step dequantises every expert with work
# once and applies it with the tensor-core GEMM instead of streaming its blocks once per group of 8 routes.
_DENSE_EXPERT_ROUTES = int(os.environ.get("FI_GGUF_MOE_DENSE_ROUTES", "64"))

PAD_HD = 256


class MLAAttention(nn.Module):
    def __init__(self, arch: ModelArch, i: int, dtype, qc, prefix: str):
        super().__init__()
        m = arch.mla
        tp = pstate.tp_size()
        self.nh_total, self.nh = arch.num_heads, arch.num_heads // tp
        self.nope, self.rope, self.vd, self.kv_lora, self.q_lora = m.qk_nope_dim, m.qk_rope_dim, m.v_head_dim, m.kv_lora_rank, m.q_lora_rank
        self.qk = self.nope + self.rope
        assert self.qk <= PAD_HD and self.vd <= PAD_HD
        H = arch.hidden_size
        if self.q_lora:
            self.q_a_proj = LiteLinear(H, self.q_lora, dtype=dtype, quant_config=qc, prefix=prefix + ".q_a_proj")
            self.q_a_layernorm = RMSNormWeight(self.q_lora, arch.rms_eps, dtype)
            self.q_b_proj = LiteLinear(self.q_lora, self.nh_total * self.qk, dtype=dtype, shard="column",
                                       quant_config=qc, prefix=prefix + ".q_b_proj")
        else:
            self.q_proj = LiteLinear(H, self.nh_total * self.qk, dtype=dtype, shard="column", quant_config=qc,
                                     prefix=prefix + ".q_proj")
        self.kv_a_proj_with_mqa = LiteLinear(H, self.kv_lora + self.rope, dtype=dtype, quant_config=qc,
                                             prefix=prefix + ".kv_a_proj_with_mqa")
        self.kv_a_layernorm = RMSNormWeight(self.kv_lora, arch.rms_eps, dtype)
        self.kv_b_proj = LiteLinear(self.kv_lora, self.nh_total * (self.nope + self.vd), dtype=dtype, shard="column",
                                    quant_config=qc, prefix=prefix + ".kv_b_proj")
        self.o_proj = LiteLinear(self.nh_total * self.vd, H, dtype=dtype, shard="row", quant_config=qc,
                                 prefix=prefix + ".o_proj")
        self.sm_scale = self.qk ** -0.5
        self.rope_theta, self.rope_scaling = arch.rope_theta, arch.rope_scaling
        self._cos_sin = None
        self.absorbed = False      # set by the model once the weights are in (see kv_cache_specs)

    def can_absorb(self) -> bool:
        """The absorbed form needs the kv_b projection as a dense 16-bit matrix on a GPU (its two halves are
        applied per head, before and after the attention) and the cache-row geometry the kernel is built for."""
        w = getattr(self.kv_b_proj, "weight", None)
        return (w is not None and w.is_cuda and w.dtype in (torch.bfloat16, torch.float16)
                and self.kv_lora == 512 and self.rope == 64 and self.kv_b_proj.bias is None)

    def _forward_absorbed(self, x, h, batch, kv, max_pos):
        """Attention over one shared cache row per token ([normed latent | rotary key], 576 values):
        q_nope goes through W_UK first (a batched product per head), the kernel returns sums of latent rows,
        W_UV is applied to them afterwards.  Prefill rows are flattened: every new token is a row with its own
        visible length."""
        T = x.shape[0]
        nh, nope, vd = self.nh, self.nope, self.vd
        if self.q_lora:
            q = self.q_b_proj(self.q_a_layernorm(self.q_a_proj(x)))
        else:
            q = self.q_proj(x)
        q = q.view(T, nh, self.qk)
        kva = self.kv_a_proj_with_mqa(x)
        cache = kv[0]
        if cache.dtype != x.dtype or cache.shape[-1] != self.kv_lora + self.rope:
            raise RuntimeError("absorbed multi-head latent attention needs a 16-bit cache of 576-value rows; "
                               "set FI_MLA_ABSORBED=0 for quantised KV caches")
        w = self.kv_b_proj.weight.view(nh, nope + vd, self.kv_lora)
        q_lat = torch.bmm(q[..., :nope].transpose(0, 1), w[:, :nope, :])          # [nh, T, 512]
        q_cat = torch.empty(T, nh, self.kv_lora + self.rope, dtype=x.dtype, device=x.device)
        lib = _lib.kernels()
        dt = ops._DT[x.dtype]
        rc = lib.fi_mla_prepare(_p(kva), kva.stride(0), _p(self.kv_a_layernorm.weight), self.kv_a_layernorm.eps, _p(q),
                                nope, _p(q_lat), q_lat.stride(0), q_lat.stride(1), _p(batch.positions),
                                _p(self.cos_sin(x.device, max_pos)), _p(batch.slot_mapping), _p(cache), _p(q_cat), T, nh,
                                dt, _stream())
        _lib.check(rc, "fi_mla_prepare")
        if not batch.is_decode:
            return self._prefill_from_latent(x, h, batch, q, q_cat, cache)
        rows, row_lens, seq_of_row = T, batch.seq_lens, None
        bs = cache.shape[2]
        chunks = max(1, (int(batch.max_kv_len) + 63) // 64)
        ctas = max(1, rows * ((nh + 15) // 16))
        splits = int(max(1, min((2 * 148 + ctas - 1) // ctas, chunks, 16)))
        ws_o = ws_ml = None
        if splits > 1:
            n_o = rows * nh * splits * self.kv_lora
            ws = scratch("mla_ws", (n_o + rows * nh * splits * 2) * 4, x.device).view(torch.float32)
            ws_o, ws_ml = ws[:n_o], ws[n_o:]
        out_lat = torch.empty(nh, T, self.kv_lora, dtype=x.dtype, device=x.device)
        rc = lib.fi_mla_decode(_p(q_cat), _p(cache), _p(out_lat), out_lat.stride(0), out_lat.stride(1),
                               _p(batch.block_tables), _p(row_lens), _p(seq_of_row), _p(ws_o), _p(ws_ml), rows, nh,
                               batch.block_tables.shape[1], bs, splits, self.sm_scale, dt, _stream())
        _lib.check(rc, "fi_mla_decode")
        _count(3 if splits > 1 else 2)
        o = torch.bmm(out_lat, w[:, nope:, :].transpose(1, 2))                      # [nh, T, vd]
        return self.o_proj(o.transpose(0, 1).reshape(T, nh * vd), residual=h, out=h)

    def _prefill_from_latent(self, x, h, batch, q, q_cat, cache):
        """Prefill of the absorbed form: many query rows per sequence make the per-head form the efficient
        one, so the context of every sequence of the batch (cached prefix + the rows just written) is gathered
        from the latent cache, up-projected through kv_b, laid out as padded per-head K/V rows in a temporary
        paged pool with consecutive blocks, and the ordinary varlen prefill kernel runs on that pool."""
        T = x.shape[0]
        nh, nope, vd, rope = self.nh, self.nope, self.vd, self.rope
        dev, dt = x.device, x.dtype
        B = batch.seq_lens.shape[0]
        bs = cache.shape[2]
        lens = batch.seq_lens.to(torch.int64)
        blocks_per = (lens + bs - 1) // bs
        blk0 = torch.cumsum(blocks_per, 0) - blocks_per                       # first temporary block of every sequence
        cu = torch.cumsum(lens, 0)
        Tc = int(sum(batch.seq_lens_cpu)) if batch.seq_lens_cpu else int(cu[-1].item())
        n_tmp = int(sum((n + bs - 1) // bs for n in batch.seq_lens_cpu)) if batch.seq_lens_cpu else int(blocks_per.sum().item())
        idx = torch.arange(Tc, device=dev)
        seq = torch.searchsorted(cu, idx, right=True)
        pos = idx - (cu - lens)[seq]
        src_blk = batch.block_tables.to(torch.int64)[seq, pos // bs]
        ctx = cache.view(-1, self.kv_lora + rope)[src_blk * bs + pos % bs]     # [Tc, 576]: normed latent | rotated key
        kvb = self.kv_b_proj(ctx[:, : self.kv_lora].contiguous())              # [Tc, nh * (nope + vd)]
        tmp_slots = ((blk0[seq] + pos // bs) * bs + pos % bs).to(torch.int32)
        pools = scratch("mla_tmp_pool", 2 * n_tmp * nh * bs * PAD_HD * x.element_size() + 512, dev)
        half = n_tmp * nh * bs * PAD_HD * x.element_size()
        k_pool = pools[:half].view(dt).view(n_tmp, nh, bs, PAD_HD)
        v_pool = pools[half:2 * half].view(dt).view(n_tmp, nh, bs, PAD_HD)
        lib = _lib.kernels()
        rc = lib.fi_mla_ctx_to_pool(_p(ctx), _p(kvb), _p(tmp_slots), _p(k_pool), _p(v_pool), Tc, nh, nope, vd, PAD_HD, bs,
                                    ops._DT[dt], _stream())
        _lib.check(rc, "fi_mla_ctx_to_pool")
        _count()
        max_b = int(max((n + bs - 1) // bs for n in batch.seq_lens_cpu)) if batch.seq_lens_cpu else int(blocks_per.max().item())
        tmp_bt = (blk0[:, None] + torch.arange(max_b, device=dev)[None, :]).clamp_(max=max(n_tmp - 1, 0)).to(torch.int32)
        q_pad = torch.zeros(T, nh, PAD_HD, dtype=dt, device=dev)
        q_pad[..., :rope] = q_cat[..., self.kv_lora:]
        q_pad[..., rope:rope + nope] = q[..., :nope]
        attn = ops.paged_attention_prefill(q_pad.view(T, nh * PAD_HD), k_pool, v_pool, tmp_bt, batch.seq_lens, batch.cu_q,
                                           batch.max_q_len, nh, nh, PAD_HD, self.sm_scale, 0, 0.0, 1.0, 1.0)
        o_in = attn.view(T, nh, PAD_HD)[..., :vd].reshape(T, nh * vd)
        return self.o_proj(o_in, residual=h, out=h)

    def cos_sin(self, device, max_pos):
        if self._cos_sin is None or self._cos_sin.device != device:
            self._cos_sin = get_cos_sin(self.rope, max_pos, self.rope_theta, None, device)
        return self._cos_sin

    def forward(self, x, h, batch, kv, max_pos):
        if self.absorbed and x.is_cuda:
            return self._forward_absorbed(x, h, batch, kv, max_pos)
        T = x.shape[0]
        if x.is_cuda and T > _MATERIALISED_MAX_TOKENS:
            # one prefill step of 16,000 tokens in this form ended in an illegal-address report on a B200 and the
            # cause has not been found; steps of up to 3,072 tokens are covered by tests
            raise RuntimeError(f"the materialised attention form takes at most {_MATERIALISED_MAX_TOKENS} tokens per "
                               f"step (got {T}): lower max_num_batched_tokens or use the absorbed form")
        if self.q_lora:
            q = self.q_b_proj(self.q_a_layernorm(self.q_a_proj(x)))
        else:
            q = self.q_proj(x)
        q = q.view(T, self.nh, self.qk)
        kva = self.kv_a_proj_with_mqa(x)
        latent = self.kv_a_layernorm(kva[:, : self.kv_lora].contiguous())
        k_rope = kva[:, self.kv_lora:]
        kvb = self.kv_b_proj(latent).view(T, self.nh, self.nope + self.vd)
        # assemble [q | k | v] with padded heads laid out [rope | nope | 0]
        if x.is_cuda and q.is_contiguous() and kvb.is_contiguous() and x.dtype in (torch.bfloat16, torch.float16):
            buf = torch.empty(T, 3 * self.nh, PAD_HD, dtype=x.dtype, device=x.device)
            rc = _lib.kernels().fi_mla_assemble(_p(q), _p(k_rope), k_rope.stride(0), _p(kvb), _p(buf), T, self.nh,
                                                self.nope, self.rope, self.vd, PAD_HD, ops._DT[x.dtype], _stream())
            _lib.check(rc, "fi_mla_assemble")
            _count()
        else:
            buf = torch.zeros(T, 3 * self.nh, PAD_HD, dtype=x.dtype, device=x.device)
            buf[:, : self.nh, : self.rope] = q[..., self.nope:]
            buf[:, : self.nh, self.rope:self.qk] = q[..., : self.nope]
            buf[:, self.nh:2 * self.nh, : self.rope] = k_rope[:, None, :]
            buf[:, self.nh:2 * self.nh, self.rope:self.qk] = kvb[..., : self.nope]
            buf[:, 2 * self.nh:, : self.vd] = kvb[..., self.nope:]
        qkv = buf.view(T, 3 * self.nh * PAD_HD)
        k_cache, v_cache = kv
        cfg = batch.config
        ops.rope_and_cache(qkv, batch.positions, self.cos_sin(x.device, max_pos), batch.slot_mapping, k_cache, v_cache,
                           self.nh, self.nh, PAD_HD, self.rope, k_scale=cfg.k_scale, v_scale=cfg.v_scale)
        if batch.is_decode:
            attn = ops.paged_attention_decode(qkv, k_cache, v_cache, *batch.attention_tables(0), self.nh,
                                              self.nh, PAD_HD, self.sm_scale, 0, 0.0, cfg.k_scale, cfg.v_scale,
                                              max_kv_len=batch.max_kv_len)
        else:
            attn = ops.paged_attention_prefill(qkv, k_cache, v_cache, batch.block_tables, batch.seq_lens, batch.cu_q,
                                               batch.max_q_len, self.nh, self.nh, PAD_HD, self.sm_scale, 0, 0.0,
                                               cfg.k_scale, cfg.v_scale)
        o_in = attn.view(T, self.nh, PAD_HD)[..., : self.vd].reshape(T, self.nh * self.vd)
        return self.o_proj(o_in, residual=h, out=h)


class GatedMLP(nn.Module):
    def __init__(self, H: int, inter: int, dtype, qc, prefix: str, act: str = "silu"):
        super().__init__()
        self.gate_up_proj = LiteLinear(H, 2 * inter, dtype=dtype, shard="column", quant_config=qc,
                                       prefix=prefix + ".gate_up_proj", gated_act=act, out_splits=[inter, inter])
        self.down_proj = LiteLinear(inter, H, dtype=dtype, shard="row", quant_config=qc, prefix=prefix + ".down_proj")

    def forward(self, x, residual=None):
        return self.down_proj(self.gate_up_proj(x), residual=residual, out=residual)


def _block_staging_budget(arch) -> int | None:
    """Device bytes one MoE block may spend on expert payloads: the model's budget (``expert_staging_gb`` of the
    architecture's extras, else ``FI_EXPERT_STAGING_GB``) split evenly over its MoE blocks.  None: no staging."""
    from ..layers import expert_stager
    total = arch.extra.get("expert_staging_gb")
    total = int(float(total) * 2 ** 30) if total else expert_stager.budget_bytes_from_env()
    if total is None:
        return None
    blocks = arch.extra.get("moe_blocks") or \
        max(1, getattr(arch, "num_layers", 1) - getattr(arch.moe, "first_dense_layers", 0))
    return max(1, total // int(blocks))


class RoutedExperts(nn.Module):
    """Routed experts kept as raw GGUF blocks: gate/up ``[E, I, row bytes]``, down ``[E, H, row bytes]``."""

    def __init__(self, arch: ModelArch, dtype):
        super().__init__()
        ep, r = pstate.ep_size(), pstate.ep_rank()
        self.E, self.I, self.H, self.top_k = arch.moe.num_experts, arch.moe.expert_intermediate, arch.hidden_size, arch.moe.top_k
        self.e_local = self.E // ep
        self.e_lo = r * self.e_local
        self.device = torch.empty(0).device
        self.dtype = dtype
        self.raw: dict[str, torch.Tensor] = {}
        self.types: dict[str, int] = {}
        self.clamp = float(arch.extra.get("swiglu_clamp", 0.0))
        # a device budget for expert payloads keeps them in pinned host memory behind a slab of device slots
        self.stage_budget = _block_staging_budget(arch)
        self.host: dict[str, torch.Tensor] = {}
        self.stager = None

    def load(self, which: str, t) -> None:
        from ..loaders.gguf import GGUFTensor
        if isinstance(t, GGUFTensor):
            blocks = t.raw[self.e_lo:self.e_lo + self.e_local].contiguous()
            self.types[which] = t.ggml_type
        else:   # float experts: store as Q8_0 blocks so one code path serves them
            w = t[self.e_lo:self.e_lo + self.e_local].float()
            E, R, K = w.shape
            blocks = gq.quantize_q8_0(w.reshape(E * R, K)).view(E, R, -1)
            self.types[which] = 8
        if self.stage_budget is None:
            self.raw[which] = blocks.to(self.device)
        else:
            blocks = blocks.cpu()
            if torch.device(self.device).type == "cuda":
                try:
                    blocks = blocks.pin_memory()
                except RuntimeError as e:     # the host refuses to lock that much: pageable copies still work, slower
                    logger.warning("expert payload %s stays in pageable host memory (%s)", which, e)
            self.host[which] = blocks
            self.stager = None

    def _ensure_stager(self):
        """Built at the first step after the three payloads arrived.  A budget that holds every expert turns
        staging off: the payloads move to the device for good."""
        if self.stager is None and len(self.host) == 3:
            from ..layers.expert_stager import ExpertStager
            per_expert = sum(int(t[0].numel()) * t.element_size() for t in self.host.values())
            if self.stage_budget >= per_expert * self.e_local:
                for k, t in self.host.items():
                    self.raw[k] = t.to(self.device)
                self.host, self.stage_budget = {}, None
                return None
            self.stager = ExpertStager(self.host, self.device, self.stage_budget, min_slots=min(self.e_local, self.top_k))
        return self.stager

    def _forward_staged(self, x, ids, weights, reduce: bool):
        """The step's experts become resident in waves; each wave runs on the slab with its routes renumbered
        to slots and every other route dropped.  One host read of the routed ids per block."""
        st = self.stager
        st.begin_step()
        named = torch.unique(ids).tolist()
        local = [e - self.e_lo for e in named if self.e_lo <= e < self.e_lo + self.e_local]
        out = None
        for wave in st.waves(local):
            placed = st.stage(wave)
            part = self._core(x, st.slot_ids(ids, placed, self.e_lo), weights, False, st.slab, 0, st.slots)
            out = part if out is None else out.add_(part)
        if out is None:
            out = torch.zeros(x.shape[0], self.H, dtype=x.dtype, device=x.device)
        if pstate.ep_size() > 1 and reduce:
            from ..parallel import fused_ops
            out = fused_ops.all_reduce_activations(out)
        return out

    def forward(self, x, ids, weights, reduce: bool = True):
        """``reduce=False``: the caller owns the exchange between the expert-parallel ranks (rows that arrived by
        all-to-all): only this rank's experts run, nothing is summed over ranks."""
        from ..parallel import ep_alltoall
        if reduce and pstate.ep_size() > 1 and ep_alltoall.ENABLED:
            def run(rows, expert_ids):
                one = torch.ones(rows.shape[0], 1, dtype=torch.float32, device=rows.device)
                return self.forward(rows, expert_ids.view(-1, 1).to(ids.dtype), one, reduce=False)
            return ep_alltoall.sharded_moe(x, ids, weights, self.e_local, run)
        if self.stage_budget is not None and self._ensure_stager() is not None:
            return self._forward_staged(x, ids, weights, reduce)
        return self._core(x, ids, weights, reduce, self.raw, self.e_lo, self.e_local)

    def _core(self, x, ids, weights, reduce, raw, e_lo, e_local):
        """The experts ``[e_lo, e_lo + e_local)`` whose payloads are ``raw`` applied to the routes that name them;
        other routes contribute nothing."""
        T, H = x.shape
        K = ids.shape[1]
        n = T * K
        if not x.is_cuda:
            out = torch.zeros(T, H, dtype=torch.float32)
            g = gq.dequantize(raw["gate"].reshape(-1, raw["gate"].shape[-1]), self.types["gate"], H).view(e_local, self.I, H)
            u = gq.dequantize(raw["up"].reshape(-1, raw["up"].shape[-1]), self.types["up"], H).view(e_local, self.I, H)
            d = gq.dequantize(raw["down"].reshape(-1, raw["down"].shape[-1]), self.types["down"], self.I).view(e_local, H, self.I)
            xf = x.float()
            for e in range(e_local):
                tok, slot = torch.nonzero(ids == e + e_lo, as_tuple=True)
                if tok.numel() == 0:
                    continue
                gv, uv = xf[tok] @ g[e].t(), xf[tok] @ u[e].t()
                if self.clamp > 0:
                    gv, uv = gv.clamp(max=self.clamp), uv.clamp(-self.clamp, self.clamp)
                a = (torch.nn.functional.silu(gv) * uv).to(x.dtype).float()
                y = (a @ d[e].t()).to(x.dtype).float()
                out.index_add_(0, tok, y * weights[tok, slot][:, None])
            out = out.to(x.dtype)
        else:
            lib = _lib.kernels()
            esz = x.element_size()
            buf = scratch("ds_moe", n * (self.I + H) * esz + 256, x.device)
            a = buf[: n * self.I * esz].view(x.dtype).view(n, self.I)
            y = buf[n * self.I * esz: n * (self.I + H) * esz].view(x.dtype).view(n, H)
            e_hi = e_lo + e_local
            ids_flat = ids.reshape(-1)
            slot_of = None
            if (reduce or raw is not self.raw) and n >= _DENSE_EXPERT_ROUTES * e_local and self.clamp <= 0 \
                    and x.dtype in (torch.bfloat16, torch.float16):
                return self._forward_tensor_core(x, ids_flat, weights, a, y, T, K, H, raw, e_lo, e_local, reduce)
            same_gu = self.types["gate"] == self.types["up"]
            # int8 activations + dp4a for the 2-bit formats; 16-bit activations for the others
            q8 = _Q8 and x.dtype == torch.bfloat16 and same_gu and self.types["gate"] in (10, 16) \
                and self.types["down"] in (10, 16)
            grouped = q8 or ((_GROUPED == "on" or (_GROUPED == "auto" and n >= e_local))
                             and x.dtype == torch.bfloat16 and same_gu and self.types["gate"] in (8, 10, 16))
            if grouped:
                # routes sorted by expert; a tile of up to 8 routes of one expert streams that expert once.  Steps
                # with fewer routes than experts (small decode batches) use tiles of one route.
                tile_m = 8 if (not q8 or n >= e_local) else 1
                max_tiles = n if tile_m == 1 else n // 8 + e_local
                ints = scratch("ds_moe_ints", (2 * n + e_local + 1 + 3 * max_tiles + 8) * 4, x.device).view(torch.int32)
                o = 0
                sorted_route = ints[o:o + n]; o += n
                slot_of = ints[o:o + n]; o += n
                offsets = ints[o:o + e_local + 1]; o += e_local + 1
                tile_expert = ints[o:o + max_tiles]; o += max_tiles
                tile_row0 = ints[o:o + max_tiles]; o += max_tiles
                tile_rows = ints[o:o + max_tiles]; o += max_tiles
                n_tiles = ints[o:o + 1]
                rc = lib.fi_moe_align(_p(ids_flat), n, e_lo, e_hi, tile_m, _p(sorted_route), _p(slot_of), _p(offsets),
                                      _p(tile_expert), _p(tile_row0), _p(tile_rows), _p(n_tiles), _stream())
                _lib.check(rc, "fi_moe_align")
                if q8:
                    rc = lib.fi_gguf_moe_gate_up_q8(
                        _p(x), x.stride(0), _p(raw["gate"]), _p(raw["up"]), self.types["gate"],
                        self.types["up"], raw["gate"].shape[-1], raw["up"].shape[-1], _p(sorted_route),
                        _p(tile_expert), _p(tile_row0), _p(tile_rows), _p(n_tiles), max_tiles, tile_m, K, self.I, H,
                        self.clamp, _p(a), _stream())
                    _lib.check(rc, "fi_gguf_moe_gate_up_q8")
                    rc = lib.fi_gguf_moe_down_q8(_p(a), _p(raw["down"]), self.types["down"],
                                                 raw["down"].shape[-1], _p(tile_expert), _p(tile_row0),
                                                 _p(tile_rows), _p(n_tiles), max_tiles, tile_m, H, self.I, _p(y),
                                                 _stream())
                    _lib.check(rc, "fi_gguf_moe_down_q8")
                else:
                    rc = lib.fi_gguf_moe_gate_up_grouped(
                        _p(x), x.stride(0), _p(raw["gate"]), _p(raw["up"]), self.types["gate"],
                        self.types["up"], raw["gate"].shape[-1], raw["up"].shape[-1], _p(sorted_route),
                        _p(tile_expert), _p(tile_row0), _p(tile_rows), _p(n_tiles), max_tiles, K, self.I, H, self.clamp,
                        _p(a), _stream())
                    _lib.check(rc, "fi_gguf_moe_gate_up_grouped")
                    rc = lib.fi_gguf_moe_down_grouped(_p(a), _p(raw["down"]), self.types["down"],
                                                      raw["down"].shape[-1], _p(tile_expert), _p(tile_row0),
                                                      _p(tile_rows), _p(n_tiles), max_tiles, H, self.I, _p(y), _stream())
                    _lib.check(rc, "fi_gguf_moe_down_grouped")
                _count(1)
            else:
                rc = lib.fi_gguf_moe_gate_up(_p(x), x.stride(0), _p(raw["gate"]), _p(raw["up"]),
                                             self.types["gate"], self.types["up"], raw["gate"].shape[-1],
                                             raw["up"].shape[-1], _p(ids_flat), n, K, e_lo, e_hi, self.I, H,
                                             self.clamp, _p(a), _stream())
                _lib.check(rc, "fi_gguf_moe_gate_up")
                rc = lib.fi_gguf_moe_down(_p(a), _p(raw["down"]), self.types["down"], raw["down"].shape[-1],
                                          _p(ids_flat), n, e_lo, e_hi, H, self.I, _p(y), _stream())
                _lib.check(rc, "fi_gguf_moe_down")
            out = torch.empty(T, H, dtype=x.dtype, device=x.device)
            heap = None
            if pstate.ep_size() > 1 and reduce:
                from ..parallel import fused_ops
                heap = fused_ops.ep_heap(x)
            if heap is not None and heap.fits_low_latency(T, H):
                # expert parallel: combine + sum over ranks in one kernel (routes of other ranks are zero rows)
                import ctypes
                comm = heap.comm_desc(mode=1, T=T, N=H, xfer_16bit=2)
                rc = lib.fi_moe_combine_allreduce(_p(y), _p(slot_of), _p(weights), None, _p(out), T, K, H, ops._DT[x.dtype],
                                                  _p(ops.status_word(x.device)), _stream(), ctypes.byref(comm))
                _lib.check(rc, "fi_moe_combine_allreduce")
                _count(3)
                return out
            rc = lib.fi_moe_combine(_p(y), _p(slot_of), _p(weights), None, _p(out), T, K, H, ops._DT[x.dtype], _stream())
            _lib.check(rc, "fi_moe_combine")
            _count(3)
        if pstate.ep_size() > 1 and reduce:
            from ..parallel import fused_ops
            out = fused_ops.all_reduce_activations(out)
        return out


    def _forward_tensor_core(self, x, ids_flat, weights, a, y, T, K, H, raw, e_lo, e_local, reduce):
        """Large prefill steps (on average dozens of routes per expert): the routes are sorted by expert, the
        activation rows gathered in that order, and every expert with work is dequantised into a 16-bit scratch
        matrix and applied with the tcgen05 GEMM (gate|up, SiLU * up, down).  Streaming the 2-bit blocks once per
        group of 8 routes (the GEMV-style kernels) costs a pass over the expert per group; here an expert is
        decoded once per step.  One host read of the per-expert route counts per layer."""
        lib = _lib.kernels()
        n = T * K
        dev, dt = x.device, x.dtype
        ints = scratch("ds_moe_ints", (2 * n + e_local + 1 + 3 * (n // 128 + e_local) + 8) * 4, dev).view(torch.int32)
        mt = n // 128 + e_local
        o = 0
        sorted_route = ints[o:o + n]; o += n
        slot_of = ints[o:o + n]; o += n
        offsets = ints[o:o + e_local + 1]; o += e_local + 1
        tile_expert = ints[o:o + mt]; o += mt
        tile_row0 = ints[o:o + mt]; o += mt
        tile_rows = ints[o:o + mt]; o += mt
        n_tiles = ints[o:o + 1]
        rc = lib.fi_moe_align(_p(ids_flat), n, e_lo, e_lo + e_local, 128, _p(sorted_route), _p(slot_of),
                              _p(offsets), _p(tile_expert), _p(tile_row0), _p(tile_rows), _p(n_tiles), _stream())
        _lib.check(rc, "fi_moe_align")
        xs = scratch("ds_moe_xs", n * H * x.element_size() + 256, dev)[: n * H * x.element_size()].view(dt).view(n, H)
        rc = lib.fi_moe_gather(_p(x), _p(sorted_route), _p(offsets), e_local, n, K, H, _p(xs), ops._DT[dt], _stream())
        _lib.check(rc, "fi_moe_gather")
        off = offsets.tolist()
        I = self.I
        wgu = scratch("ds_moe_wgu", 2 * I * H * 2 + 256, dev)[: 2 * I * H * 2].view(dt).view(2 * I, H)
        wd = scratch("ds_moe_wd", H * I * 2 + 256, dev)[: H * I * 2].view(dt).view(H, I)
        gu = scratch("ds_moe_gu", max(off[e + 1] - off[e] for e in range(e_local)) * 2 * I * 2 + 256, dev)
        for e in range(e_local):
            r0, r1 = off[e], off[e + 1]
            if r1 <= r0:
                continue
            gq.dequantize_cuda(raw["gate"][e], self.types["gate"], H, dt, out=wgu[:I])
            gq.dequantize_cuda(raw["up"][e], self.types["up"], H, dt, out=wgu[I:])
            g = gu[: (r1 - r0) * 2 * I * 2].view(dt).view(r1 - r0, 2 * I)
            ops.linear(xs[r0:r1], wgu, out=g, static_weight=False)
            ops.act_mul(g, "silu", out=a[r0:r1])
            gq.dequantize_cuda(raw["down"][e], self.types["down"], I, dt, out=wd)
            ops.linear(a[r0:r1], wd, out=y[r0:r1], static_weight=False)
        out = torch.empty(T, H, dtype=dt, device=dev)
        rc = lib.fi_moe_combine(_p(y), _p(slot_of), _p(weights), None, _p(out), T, K, H, ops._DT[dt], _stream())
        _lib.check(rc, "fi_moe_combine")
        _count(3)
        if pstate.ep_size() > 1 and reduce:
            from ..parallel import fused_ops
            out = fused_ops.all_reduce_activations(out)
        return out


class DeepseekMoE(nn.Module):
    def __init__(self, arch: ModelArch, dtype, qc, prefix: str):
        super().__init__()
        E, H = arch.moe.num_experts, arch.hidden_size
        self.gate = nn.Parameter(torch.empty(E, H, dtype=dtype), requires_grad=False)
        self.e_score_correction_bias = nn.Parameter(torch.zeros(E, dtype=torch.float32), requires_grad=False)
        self.experts = RoutedExperts(arch, dtype)
        self.mode, self.renorm, self.scale, self.top_k = arch.moe.router, arch.moe.renormalize, arch.moe.routed_scaling, arch.moe.top_k
        self.shared_experts = GatedMLP(H, arch.moe.shared_intermediate, dtype, qc, prefix + ".shared_experts") \
            if arch.moe.shared_intermediate else None

    def forward(self, x, h):
        logits = ops.linear(x, self.gate, out_dtype=torch.float32)
        bias = self.e_score_correction_bias if self.mode != "softmax" else None
        ids, w = moe_ops.route(logits, self.top_k, self.mode, bias, None, self.renorm, self.scale)
        routed = self.experts(x, ids, w)
        if self.shared_experts is not None:
            h = self.shared_experts(x, residual=h)
        return h.add_(routed) if h.is_cuda or True else h + routed


class DeepseekDecoderLayer(nn.Module):
    def __init__(self, arch: ModelArch, i: int, dtype, qc):
        super().__init__()
        p = f"model.layers.{i}"
        self.input_layernorm = RMSNormWeight(arch.hidden_size, arch.rms_eps, dtype)
        self.post_attention_layernorm = RMSNormWeight(arch.hidden_size, arch.rms_eps, dtype)
        self.self_attn = MLAAttention(arch, i, dtype, qc, p + ".self_attn")
        self.is_moe = arch.moe.num_experts > 0 and i >= arch.moe.first_dense_layers
        if self.is_moe:
            self.mlp = DeepseekMoE(arch, dtype, qc, p + ".mlp")
        else:
            self.mlp = GatedMLP(arch.hidden_size, arch.intermediate_size, dtype, qc, p + ".mlp")

    def forward(self, h, batch, kv, max_pos):
        with stage("layer.attention"):
            h = self.self_attn(self.input_layernorm(h), h, batch, kv, max_pos)
        x = self.post_attention_layernorm(h)
        with stage("layer.moe" if self.is_moe else "layer.mlp"):
            if self.is_moe:
                return self.mlp(x, h)
            return self.mlp(x, residual=h)


class DeepseekMLAForCausalLM(nn.Module):
    supports_lora = False
    supports_multimodal = False

    def __init__(self, vllm_config):
        super().__init__()
        mc = vllm_config.model_config
        arch: ModelArch = mc.arch
        self.arch, self.dtype = arch, mc.dtype
        qc = vllm_config.quant_config
        from ..parallel import ep_alltoall
        if ep_alltoall.ENABLED and pstate.ep_size() > 1:
            self.supports_cuda_graph = False      # the all-to-all split sizes are read on the host every step
        if arch.moe is not None and _block_staging_budget(arch) is not None:
            self.supports_cuda_graph = False      # staged experts: the routed ids are read on the host every block
        self.embed_tokens = nn.Parameter(torch.empty(arch.vocab_size, arch.hidden_size, dtype=mc.dtype), requires_grad=False)
        self.layers = nn.ModuleList([DeepseekDecoderLayer(arch, i, mc.dtype, qc) for i in range(arch.num_layers)])
        self.norm = RMSNormWeight(arch.hidden_size, arch.rms_eps, mc.dtype)
        self.lm_head = LiteLinear(arch.hidden_size, arch.vocab_size, dtype=mc.dtype, shard="column",
                                  quant_config=qc, prefix="lm_head")
        self.max_pos = max(mc.max_model_len, 16)

    def kv_cache_specs(self):
        """Called once the weights are in.  With dense 16-bit kv_b projections on a GPU the attention runs in
        absorbed form on one shared [latent | rotary key] row per token (576 values, no V pool); otherwise
        per-head K and V rows padded to 256 channels."""
        from ..engine.kv_cache import KVLayerSpec
        for l in self.layers:
            qm = getattr(l.self_attn.kv_b_proj, "quant_method", None)
            if qm is not None and hasattr(qm, "process_weights_after_loading"):
                qm.process_weights_after_loading(l.self_attn.kv_b_proj)
        absorb = _ABSORBED and all(l.self_attn.can_absorb() for l in self.layers)
        for l in self.layers:
            l.self_attn.absorbed = absorb
        if absorb:
            a = self.layers[0].self_attn
            return [KVLayerSpec(1, a.kv_lora + a.rope, 0) for _ in self.layers]
        return [(l.self_attn.nh, PAD_HD) for l in self.layers]

    def forward(self, batch, kv_caches, inputs_embeds=None):
        h = inputs_embeds if inputs_embeds is not None else ops.embedding(batch.input_ids, self.embed_tokens)
        for i, layer in enumerate(self.layers):
            h = layer(h, batch, kv_caches[i], self.max_pos)
        last = h if batch.logits_indices is None else h.index_select(0, batch.logits_indices)
        logits = self.lm_head(self.norm(last), out_dtype=torch.float32)
        if self.lm_head.tp > 1:
            logits = pstate.all_gather_last_dim(logits)
        return logits

    def load_weights(self, weights):
        from ..loaders.gguf import GGUFTensor
        from ..loaders.weight_utils import finalize_quantized, load_mapped
        m: dict = {"model.norm": ("norm", self.norm), "lm_head": ("linear", self.lm_head, 0, None)}

        def load_embed(suffix, t):
            w = gq.dequantize(t.raw, t.ggml_type, t.shape[-1]) if isinstance(t, GGUFTensor) else t
            self.embed_tokens.data.copy_(w.to(self.embed_tokens.dtype))
        m["model.embed_tokens"] = ("custom", load_embed)
        for i, L in enumerate(self.layers):
            p = f"model.layers.{i}."
            at = L.self_attn
            m[p + "input_layernorm"] = ("norm", L.input_layernorm)
            m[p + "post_attention_layernorm"] = ("norm", L.post_attention_layernorm)
            for n in ("q_a_proj", "q_b_proj", "q_proj", "kv_a_proj_with_mqa", "kv_b_proj", "o_proj"):
                if hasattr(at, n):
                    m[p + "self_attn." + n] = ("linear", getattr(at, n), 0, None)
            if at.q_lora:
                m[p + "self_attn.q_a_layernorm"] = ("norm", at.q_a_layernorm)
            m[p + "self_attn.kv_a_layernorm"] = ("norm", at.kv_a_layernorm)
            if L.is_moe:
                mo = L.mlp
                m[p + "mlp.gate"] = ("custom", lambda s, t, mo=mo: (mo.gate.data.copy_(t.to(mo.gate.dtype)) if s == "weight"
                                                                   else mo.e_score_correction_bias.data.copy_(t.float())))
                for w in ("gate", "up", "down"):
                    m[p + f"mlp.experts.{w}_proj"] = ("custom", lambda s, t, X=mo.experts, w=w: X.load(w, t))
                if mo.shared_experts is not None:
                    se = mo.shared_experts
                    m[p + "mlp.shared_experts.gate_proj"] = ("linear", se.gate_up_proj, 0, None)
                    m[p + "mlp.shared_experts.up_proj"] = ("linear", se.gate_up_proj, 1, None)
                    m[p + "mlp.shared_experts.down_proj"] = ("linear", se.down_proj, 0, None)
            else:
                m[p + "mlp.gate_proj"] = ("linear", L.mlp.gate_up_proj, 0, None)
                m[p + "mlp.up_proj"] = ("linear", L.mlp.gate_up_proj, 1, None)
                m[p + "mlp.down_proj"] = ("linear", L.mlp.down_proj, 0, None)
        consumed = load_mapped(m, weights)
        finalize_quantized(self)
        return consumed
