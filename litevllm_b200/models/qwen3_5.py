"""Qwen3.5 / Qwen3-Next style hybrid decoder: three of every four layers are GatedDeltaNet linear
attention, every fourth is gated full attention.

Linear-attention layer (per token t, per value head):
  qkv = SiLU(causal depthwise conv1d_k4(in_proj_qkv(x)));  q, k L2-normalised, q scaled by dk^-0.5
  beta = sigmoid(in_proj_b(x));  g = -exp(A_log) * softplus(in_proj_a(x) + dt_bias)
  S <- S * exp(g);  delta = (v - S^T k) * beta;  S <- S + k (x) delta;  o = S^T q
  out = out_proj( RMSNorm(o) * w * SiLU(in_proj_z(x)) )
The recurrent state S [value heads, dk, dv] and the last three conv inputs are carried per request
between steps (``RequestState.linear_attn_carry`` / ``linear_conv_carry``).
Full-attention layer: q_proj emits [q | gate] per head, per-head (1+w) RMSNorm on q and k, partial
rotary (first 25 % of the head), paged attention, output multiplied by sigmoid(gate).
The recurrent rule runs in PyTorch (token loop, vectorised over heads); everything else uses the
engine's kernels.  Because of the Python-side state the decode step is not graph-captured.
Reference: vllm/model_executor/models/qwen3_5.py:42-1573.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops
from ..layers.linear import LiteLinear
from ..layers.rope import get_cos_sin
from ..parallel import state as pstate
from .arch import ModelArch
from .llama import LlamaMLP, RMSNormWeight


class GatedDeltaNet(nn.Module):
    def __init__(self, arch: ModelArch, i: int, dtype, qc, prefix: str):
        super().__init__()
        e = arch.extra
        self.nk = int(e.get("linear_num_key_heads", 4))
        self.nv = int(e.get("linear_num_value_heads", 8))
        self.dk = int(e.get("linear_key_head_dim", 64))
        self.dv = int(e.get("linear_value_head_dim", 64))
        self.kw = int(e.get("linear_conv_kernel_dim", 4))
        H = arch.hidden_size
        self.qkv_dim = 2 * self.nk * self.dk + self.nv * self.dv
        self.in_proj_qkv = LiteLinear(H, self.qkv_dim, dtype=dtype, quant_config=qc, prefix=prefix + ".in_proj_qkv")
        self.in_proj_z = LiteLinear(H, self.nv * self.dv, dtype=dtype, quant_config=qc, prefix=prefix + ".in_proj_z")
        self.in_proj_ba = LiteLinear(H, 2 * self.nv, dtype=dtype, prefix="", out_splits=[self.nv, self.nv])
        self.conv_weight = nn.Parameter(torch.empty(self.qkv_dim, self.kw, dtype=dtype), requires_grad=False)
        self.A_log = nn.Parameter(torch.zeros(self.nv, dtype=torch.float32), requires_grad=False)
        self.dt_bias = nn.Parameter(torch.zeros(self.nv, dtype=torch.float32), requires_grad=False)
        self.norm = RMSNormWeight(self.dv, arch.rms_eps, dtype)
        self.out_proj = LiteLinear(self.nv * self.dv, H, dtype=dtype, shard=None, quant_config=qc, prefix=prefix + ".out_proj")
        self.eps = arch.rms_eps

    def init_state(self, device, dtype):
        return (torch.zeros(self.nv, self.dk, self.dv, dtype=torch.float32, device=device),
                torch.zeros(self.qkv_dim, self.kw - 1, dtype=dtype, device=device))

    def forward(self, x, h, batch, carries):
        """x [T, H]; carries: list (one per sequence) of (S, conv_state) for this layer, updated in place."""
        qkv_all = self.in_proj_qkv(x)
        z_all = self.in_proj_z(x)
        ba = self.in_proj_ba(x).float()
        beta_all = torch.sigmoid(ba[:, : self.nv])
        g_all = -torch.exp(self.A_log) * F.softplus(ba[:, self.nv:] + self.dt_bias)
        outs = torch.empty(x.shape[0], self.nv * self.dv, dtype=x.dtype, device=x.device)
        rep = self.nv // self.nk
        off = 0
        for b, n in enumerate(batch.q_lens_cpu if not batch.is_decode else [1] * len(carries)):
            S, conv = carries[b]
            seq = qkv_all[off:off + n]
            ctx = torch.cat([conv.t(), seq], dim=0)                      # [kw-1+n, C]
            win = ctx.unfold(0, self.kw, 1)                               # [n, C, kw]
            mixed = F.silu((win.float() * self.conv_weight.float()).sum(-1))
            carries[b] = (S, ctx[-(self.kw - 1):].t().contiguous())
            q = mixed[:, : self.nk * self.dk].view(n, self.nk, self.dk)
            k = mixed[:, self.nk * self.dk: 2 * self.nk * self.dk].view(n, self.nk, self.dk)
            v = mixed[:, 2 * self.nk * self.dk:].view(n, self.nv, self.dv)
            q = F.normalize(q, dim=-1) * self.dk ** -0.5
            k = F.normalize(k, dim=-1)
            q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
            o = torch.empty(n, self.nv, self.dv, dtype=torch.float32, device=x.device)
            for t in range(n):
                S = S * torch.exp(g_all[off + t])[:, None, None]
                mem = torch.einsum("hkv,hk->hv", S, k[t])
                delta = (v[t] - mem) * beta_all[off + t][:, None]
                S = S + k[t][:, :, None] * delta[:, None, :]
                o[t] = torch.einsum("hkv,hk->hv", S, q[t])
            carries[b] = (S, carries[b][1])
            on = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + self.eps) * self.norm.weight.float()
            gate = F.silu(z_all[off:off + n].float().view(n, self.nv, self.dv))
            outs[off:off + n] = (on * gate).reshape(n, -1).to(x.dtype)
            off += n
        if batch.is_decode and outs.shape[0] > off:
            outs[off:] = 0
        return self.out_proj(outs, residual=h, out=h)


class GatedFullAttention(nn.Module):
    def __init__(self, arch: ModelArch, i: int, dtype, qc, prefix: str):
        super().__init__()
        self.nh, self.nkv, self.hd = arch.num_heads, arch.num_kv_heads, arch.head_dim
        H = arch.hidden_size
        self.gated = bool(arch.extra.get("attn_output_gate", True))
        q_out = self.nh * self.hd * (2 if self.gated else 1)
        self.q_proj = LiteLinear(H, q_out, dtype=dtype, quant_config=qc, prefix=prefix + ".q_proj")
        self.kv_proj = LiteLinear(H, 2 * self.nkv * self.hd, dtype=dtype, quant_config=qc, prefix=prefix + ".kv_proj",
                                  out_splits=[self.nkv * self.hd, self.nkv * self.hd])
        self.o_proj = LiteLinear(self.nh * self.hd, H, dtype=dtype, quant_config=qc, prefix=prefix + ".o_proj")
        self.q_norm = RMSNormWeight(self.hd, arch.rms_eps, dtype, plus_one=True)
        self.k_norm = RMSNormWeight(self.hd, arch.rms_eps, dtype, plus_one=True)
        self.rot_dim = max(2, int(self.hd * arch.partial_rotary_factor) // 2 * 2)
        self.rope_theta, self.eps = arch.rope_theta, arch.rms_eps
        self._cs = None

    def forward(self, x, h, batch, kv, max_pos):
        T = x.shape[0]
        qg = self.q_proj(x).view(T, self.nh, -1)
        q = qg[..., : self.hd]
        kvp = self.kv_proj(x)
        qkv = torch.cat([q.reshape(T, -1), kvp], dim=1).contiguous()
        if self._cs is None or self._cs.device != x.device:
            self._cs = get_cos_sin(self.rot_dim, max_pos, self.rope_theta, None, x.device)
        k_cache, v_cache = kv
        cfg = batch.config
        ops.rope_and_cache(qkv, batch.positions, self._cs, batch.slot_mapping, k_cache, v_cache, self.nh, self.nkv,
                           self.hd, self.rot_dim, q_norm_w=self.q_norm.weight, k_norm_w=self.k_norm.weight,
                           qk_norm_mode=1, eps=self.eps, k_scale=cfg.k_scale, v_scale=cfg.v_scale)
        if batch.is_decode:
            attn = ops.paged_attention_decode(qkv, k_cache, v_cache, batch.block_tables, batch.seq_lens, self.nh,
                                              self.nkv, self.hd, self.hd ** -0.5, 0, 0.0, cfg.k_scale, cfg.v_scale,
                                              max_kv_len=batch.max_kv_len)
        else:
            attn = ops.paged_attention_prefill(qkv, k_cache, v_cache, batch.block_tables, batch.seq_lens, batch.cu_q,
                                               batch.max_q_len, self.nh, self.nkv, self.hd, self.hd ** -0.5, 0, 0.0,
                                               cfg.k_scale, cfg.v_scale)
        if self.gated:
            gate = torch.sigmoid(qg[..., self.hd:].float()).reshape(T, -1)
            attn = (attn.float() * gate).to(x.dtype)
        return self.o_proj(attn, residual=h, out=h)


class Qwen35DecoderLayer(nn.Module):
    def __init__(self, arch: ModelArch, i: int, dtype, qc):
        super().__init__()
        p = f"model.layers.{i}"
        self.is_linear = arch.layer_type(i) == "linear"
        self.input_layernorm = RMSNormWeight(arch.hidden_size, arch.rms_eps, dtype, plus_one=True)
        self.post_attention_layernorm = RMSNormWeight(arch.hidden_size, arch.rms_eps, dtype, plus_one=True)
        if self.is_linear:
            self.linear_attn = GatedDeltaNet(arch, i, dtype, qc, p + ".linear_attn")
        else:
            self.self_attn = GatedFullAttention(arch, i, dtype, qc, p + ".self_attn")
        self.mlp = LlamaMLP(arch, dtype, qc, p + ".mlp")


class Qwen35ForCausalLM(nn.Module):
    supports_lora = False
    supports_multimodal = False
    supports_cuda_graph = False

    def __init__(self, vllm_config):
        super().__init__()
        mc = vllm_config.model_config
        arch: ModelArch = mc.arch
        assert pstate.tp_size() == 1, "the Qwen3.5 hybrid model runs on a single GPU"
        self.arch, self.dtype = arch, mc.dtype
        qc = vllm_config.quant_config
        self.embed_tokens = nn.Parameter(torch.empty(arch.vocab_size, arch.hidden_size, dtype=mc.dtype), requires_grad=False)
        self.layers = nn.ModuleList([Qwen35DecoderLayer(arch, i, mc.dtype, qc) for i in range(arch.num_layers)])
        self.norm = RMSNormWeight(arch.hidden_size, arch.rms_eps, mc.dtype, plus_one=True)
        self.lm_head = LiteLinear(arch.hidden_size, arch.vocab_size, dtype=mc.dtype, prefix="lm_head")
        self.max_pos = max(mc.max_model_len, 16)
        self.linear_idx = [i for i, l in enumerate(self.layers) if l.is_linear]

    def kv_cache_specs(self):
        # linear layers keep no KV; a zero-head spec keeps layer indexing uniform
        return [(0 if l.is_linear else self.arch.num_kv_heads, self.arch.head_dim) for l in self.layers]

    # ---- per-request recurrent state, gathered before and written back after each forward
    def prepare_batch(self, batch, states) -> None:
        dev, dt = self.embed_tokens.device, self.dtype
        carries = []
        for rid in batch.request_ids:
            st = states[rid]
            if st.linear_attn_carry is None:
                st.linear_attn_carry = {i: self.layers[i].linear_attn.init_state(dev, dt) for i in self.linear_idx}
            carries.append(st.linear_attn_carry)
        batch.extras["carries"] = carries

    def finish_batch(self, batch, states) -> None:
        batch.extras.pop("carries", None)

    def forward(self, batch, kv_caches, inputs_embeds=None):
        h = inputs_embeds if inputs_embeds is not None else ops.embedding(batch.input_ids, self.embed_tokens)
        carries = batch.extras["carries"]
        for i, layer in enumerate(self.layers):
            x = layer.input_layernorm(h)
            if layer.is_linear:
                per_seq = [c[i] for c in carries]
                h = layer.linear_attn(x, h, batch, per_seq)
                for c, new in zip(carries, per_seq):
                    c[i] = new
            else:
                h = layer.self_attn(x, h, batch, kv_caches[i], self.max_pos)
            h = layer.mlp(layer.post_attention_layernorm(h), h, batch)
        last = h if batch.logits_indices is None else h.index_select(0, batch.logits_indices)
        if batch.is_decode:
            last = last[: len(batch.request_ids)]
        return self.lm_head(self.norm(last), out_dtype=torch.float32)

    def load_weights(self, weights):
        from ..loaders.weight_utils import finalize_quantized, load_mapped
        m: dict = {"model.embed_tokens": ("param", self.embed_tokens), "model.norm": ("norm", self.norm),
                   "lm_head": ("linear", self.lm_head, 0, None)}
        for i, L in enumerate(self.layers):
            p = f"model.layers.{i}."
            m[p + "input_layernorm"] = ("norm", L.input_layernorm)
            m[p + "post_attention_layernorm"] = ("norm", L.post_attention_layernorm)
            m[p + "mlp.gate_proj"] = ("linear", L.mlp.gate_up_proj, 0, None)
            m[p + "mlp.up_proj"] = ("linear", L.mlp.gate_up_proj, 1, None)
            m[p + "mlp.down_proj"] = ("linear", L.mlp.down_proj, 0, None)
            if L.is_linear:
                la = L.linear_attn
                m[p + "linear_attn.in_proj_qkv"] = ("linear", la.in_proj_qkv, 0, None)
                m[p + "linear_attn.in_proj_z"] = ("linear", la.in_proj_z, 0, None)
                m[p + "linear_attn.in_proj_b"] = ("linear", la.in_proj_ba, 0, None)
                m[p + "linear_attn.in_proj_a"] = ("linear", la.in_proj_ba, 1, None)
                m[p + "linear_attn.out_proj"] = ("linear", la.out_proj, 0, None)
                m[p + "linear_attn.norm"] = ("norm", la.norm)

                def misc(suffix, t, la=la):
                    if suffix == "A_log":
                        la.A_log.data.copy_(t.float())
                    elif suffix == "dt_bias":
                        la.dt_bias.data.copy_(t.float())
                m[p + "linear_attn"] = ("custom", misc)
                m[p + "linear_attn.conv1d"] = ("custom", lambda s, t, la=la: la.conv_weight.data.copy_(
                    t.reshape(la.qkv_dim, la.kw).to(la.conv_weight.dtype)) if s == "weight" else None)
            else:
                sa = L.self_attn
                m[p + "self_attn.q_proj"] = ("linear", sa.q_proj, 0, None)
                m[p + "self_attn.k_proj"] = ("linear", sa.kv_proj, 0, None)
                m[p + "self_attn.v_proj"] = ("linear", sa.kv_proj, 1, None)
                m[p + "self_attn.o_proj"] = ("linear", sa.o_proj, 0, None)
                m[p + "self_attn.q_norm"] = ("norm", sa.q_norm)
                m[p + "self_attn.k_norm"] = ("norm", sa.k_norm)
        consumed = load_mapped(m, weights)
        finalize_quantized(self)
        return consumed
