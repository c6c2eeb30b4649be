"""Llama / Qwen2 / Qwen3 dense decoder (TinyLlama, the 9B AWQ config).

Pre-norm blocks on a flattened varlen token stream ``[T, hidden]``:
  RMSNorm -> merged QKV GEMM -> fused RoPE + KV-cache write -> paged attention ->
  o_proj GEMM with the residual add in its epilogue -> RMSNorm -> gated gate|up GEMM
  (SiLU*up in the epilogue) -> down GEMM (+residual).
Only the last token of every sequence reaches the lm_head.
Reference: vllm/model_executor/models/llama.py:30-319 (separate q/k/v and gate/up launches, paged
decode kernel reused for prefill), vllm/model_executor/models/qwen2.py.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..layers.linear import LiteLinear
from ..layers.rope import get_cos_sin
from ..parallel import state as pstate
from ..utils.profiling import stage
from .arch import ModelArch


class RMSNormWeight(nn.Module):
    def __init__(self, dim: int, eps: float, dtype, plus_one: bool = False):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype), requires_grad=False)
        self.eps = eps
        self.w_mode = 1 if plus_one else 0
        self.folded = False      # True: the weight lives in the following linear layers (w_mode 2 = no weight)

    def forward(self, x, out=None):
        return ops.rmsnorm(x, self.weight, self.eps, w_mode=2 if self.folded else self.w_mode, out=out)

    def weighted(self, x):
        """The full norm including its weight, whether or not the weight was folded away."""
        return ops.rmsnorm(x, self.weight, self.eps, w_mode=self.w_mode)


class LlamaAttention(nn.Module):
    def __init__(self, arch: ModelArch, layer_idx: int, dtype, quant_config, prefix: str):
        super().__init__()
        tp = pstate.tp_size()
        self.layer_idx = layer_idx
        self.hd = arch.head_dim
        self.total_heads, self.total_kv = arch.num_heads, arch.num_kv_heads
        assert self.total_heads % tp == 0, "attention heads must divide the tensor-parallel size"
        self.nh = self.total_heads // tp
        self.kv_replicas = max(1, tp // self.total_kv)
        self.nkv = max(1, self.total_kv // tp)
        self.rot_dim = arch.rotary_dim or arch.head_dim
        self.sm_scale = self.hd ** -0.5
        self.window = arch.sliding_window if arch.layer_type(layer_idx) == "sliding" else 0
        q_rows, kv_rows = self.total_heads * self.hd, self.total_kv * self.hd
        # the merged weight is sharded by hand (KV heads may be replicated), so shard=None here
        self.qkv_proj = LiteLinear(arch.hidden_size, (self.nh + 2 * self.nkv) * self.hd, bias=arch.attn_bias,
                                   dtype=dtype, quant_config=quant_config, prefix=prefix + ".qkv_proj",
                                   out_splits=[self.nh * self.hd, self.nkv * self.hd, self.nkv * self.hd])
        self.o_proj = LiteLinear(q_rows, arch.hidden_size, bias=False, dtype=dtype, shard="row",
                                 quant_config=quant_config, prefix=prefix + ".o_proj")
        self.qk_norm = arch.qk_norm
        import os
        self.fuse_rope = os.environ.get("FI_FUSE_ROPE", "1") != "0"
        if self.qk_norm:
            self.q_norm = RMSNormWeight(self.hd, arch.rms_eps, dtype, arch.norm_plus_one)
            self.k_norm = RMSNormWeight(self.hd, arch.rms_eps, dtype, arch.norm_plus_one)
        self.eps = arch.rms_eps

    def qkv_source_rows(self, which: str) -> tuple[int, int]:
        """Row range of this rank inside the full q / k / v projection."""
        r = pstate.tp_rank()
        if which == "q":
            return r * self.nh * self.hd, self.nh * self.hd
        head0 = (r // self.kv_replicas) * self.nkv
        return head0 * self.hd, self.nkv * self.hd

    def _fused_rope_ok(self, x, batch, k_cache) -> bool:
        """Decode-sized batches of plain Llama attention: rotary + cache write ride in the qkv GEMM."""
        qp = self.qkv_proj
        return (self.fuse_rope and batch.is_decode and batch.lora_mapping is None and qp.quant_method is None
                and not self.qk_norm and batch.positions.dim() == 1
                and ops.qkv_rope_cache_supported(x, qp.weight, k_cache, self.nh, self.nkv, self.hd, self.rot_dim))

    def forward(self, x, h, batch, kv, cos_sin, norm_eps: float = 0.0, lora_x=None):
        k_cache, v_cache = kv
        cfg = batch.config
        if self._fused_rope_ok(x, batch, k_cache):
            qkv = ops.linear_rope_cache(x, self.qkv_proj.weight, self.qkv_proj.bias, batch.positions, cos_sin,
                                        batch.slot_mapping, k_cache, v_cache, self.nh, self.nkv, self.hd, norm_eps)
        else:
            qkv = self.qkv_proj(x, lora_mapping=batch.lora_mapping, norm_eps=norm_eps, lora_x=lora_x)
            ops.rope_and_cache(qkv, batch.positions, cos_sin, batch.slot_mapping, k_cache, v_cache, self.nh,
                               self.nkv, self.hd, self.rot_dim,
                               q_norm_w=self.q_norm.weight if self.qk_norm else None,
                               k_norm_w=self.k_norm.weight if self.qk_norm else None,
                               qk_norm_mode=(self.q_norm.w_mode if self.qk_norm else -1), eps=self.eps,
                               k_scale=cfg.k_scale, v_scale=cfg.v_scale,
                               freq_stream=batch.extras.get("freq_stream") if batch.positions.dim() == 2 else None)
        if batch.is_decode:
            attn = ops.paged_attention_decode(qkv, k_cache, v_cache, *batch.attention_tables(self.window),
                                              self.nh, self.nkv, self.hd, self.sm_scale, self.window, 0.0,
                                              cfg.k_scale, cfg.v_scale, max_kv_len=batch.max_kv_len)
        else:
            attn = ops.paged_attention_prefill(qkv, k_cache, v_cache, batch.block_tables, batch.seq_lens,
                                               batch.cu_q, batch.max_q_len, self.nh, self.nkv, self.hd,
                                               self.sm_scale, self.window, 0.0, cfg.k_scale, cfg.v_scale)
        return self.o_proj(attn, residual=h, out=h, lora_mapping=batch.lora_mapping)


class LlamaMLP(nn.Module):
    def __init__(self, arch: ModelArch, dtype, quant_config, prefix: str):
        super().__init__()
        inter = arch.intermediate_size
        self.gate_up_proj = LiteLinear(arch.hidden_size, 2 * inter, dtype=dtype, shard="column",
                                       quant_config=quant_config, prefix=prefix + ".gate_up_proj",
                                       gated_act=arch.act, out_splits=[inter, inter])
        self.down_proj = LiteLinear(inter, arch.hidden_size, dtype=dtype, shard="row",
                                    quant_config=quant_config, prefix=prefix + ".down_proj")

    def forward(self, x, h, batch, norm_eps: float = 0.0, lora_x=None):
        a = self.gate_up_proj(x, lora_mapping=batch.lora_mapping, norm_eps=norm_eps, lora_x=lora_x)
        return self.down_proj(a, residual=h, out=h, lora_mapping=batch.lora_mapping)


class LlamaDecoderLayer(nn.Module):
    def __init__(self, arch: ModelArch, layer_idx: int, dtype, quant_config):
        super().__init__()
        prefix = f"model.layers.{layer_idx}"
        self.input_layernorm = RMSNormWeight(arch.hidden_size, arch.rms_eps, dtype, arch.norm_plus_one)
        self.self_attn = LlamaAttention(arch, layer_idx, dtype, quant_config, prefix + ".self_attn")
        self.post_attention_layernorm = RMSNormWeight(arch.hidden_size, arch.rms_eps, dtype, arch.norm_plus_one)
        self.mlp = LlamaMLP(arch, dtype, quant_config, prefix + ".mlp")

        self.fused_norm = False

    def fold_norms(self) -> None:
        """Move both RMSNorm weights into the linear layers they feed, so that on a GPU the norms run
        inside the qkv and gate|up GEMM kernels (two launches fewer per layer)."""
        if self.input_layernorm.folded or self.post_attention_layernorm.folded:
            return
        qkv, gu = self.self_attn.qkv_proj, self.mlp.gate_up_proj
        if qkv.quant_method is not None or gu.quant_method is not None or qkv.in_features % 64 or gu.in_features % 64:
            return
        qkv.fold_input_norm(self.input_layernorm.weight, self.input_layernorm.w_mode == 1)
        gu.fold_input_norm(self.post_attention_layernorm.weight, self.post_attention_layernorm.w_mode == 1)
        self.input_layernorm.folded = self.post_attention_layernorm.folded = True
        self.fused_norm = True

    def forward(self, h, batch, kv, cos_sin):
        # decode-sized batches: norms inside the GEMMs; prefill tiles are compute-bound and keep the norm kernel
        if self.fused_norm and h.is_cuda and batch.lora_mapping is None and h.shape[0] <= 64:
            h = self.self_attn(h, h, batch, kv, cos_sin, norm_eps=self.input_layernorm.eps)
            return self.mlp(h, h, batch, norm_eps=self.post_attention_layernorm.eps)
        lora = batch.lora_mapping is not None and self.fused_norm
        with stage("layer.attention"):
            x = self.input_layernorm(h)
            h = self.self_attn(x, h, batch, kv, cos_sin, lora_x=self.input_layernorm.weighted(h) if lora else None)
        with stage("layer.mlp"):
            x = self.post_attention_layernorm(h)
            return self.mlp(x, h, batch, lora_x=self.post_attention_layernorm.weighted(h) if lora else None)


class LlamaForCausalLM(nn.Module):
    supports_lora = True
    supports_multimodal = False

    def __init__(self, vllm_config):
        super().__init__()
        mc = vllm_config.model_config
        arch: ModelArch = mc.arch
        self.arch, self.dtype = arch, mc.dtype
        qc = vllm_config.quant_config
        self.embed_tokens = nn.Parameter(torch.empty(arch.vocab_size, arch.hidden_size, dtype=mc.dtype),
                                         requires_grad=False)
        self.layers = nn.ModuleList([LlamaDecoderLayer(arch, i, mc.dtype, qc) for i in range(arch.num_layers)])
        self.norm = RMSNormWeight(arch.hidden_size, arch.rms_eps, mc.dtype, arch.norm_plus_one)
        self.tie = arch.tie_embeddings
        import os
        # RMSNorm inside the qkv / gate|up GEMMs (dense 16-bit weights only); FI_FUSE_RMSNORM=0 keeps the norms apart
        self.fuse_rmsnorm = os.environ.get("FI_FUSE_RMSNORM", "1") != "0" and mc.dtype in (torch.bfloat16, torch.float16)
        if not self.tie:
            self.lm_head = LiteLinear(arch.hidden_size, arch.vocab_size, dtype=mc.dtype, shard="column",
                                      prefix="lm_head")
        self.max_pos = max(mc.max_model_len, 16)
        self._cos_sin = None
        # prefill batches of at least this many tokens run sequence-parallel under tensor parallelism
        self.sp_min_tokens = int(os.environ.get("FI_SP_MIN_TOKENS", "2048"))
        self.sp_int4 = os.environ.get("FI_SP_INT4", "0") == "1"

    # ------------------------------------------------------------------ runtime
    def cos_sin(self, device):
        if self._cos_sin is None or self._cos_sin.device != device:
            a = self.arch
            self._cos_sin = get_cos_sin(a.rotary_dim or a.head_dim, self.max_pos, a.rope_theta,
                                        a.rope_scaling, device)
        return self._cos_sin

    def kv_cache_specs(self):
        """Per layer (n_kv_heads on this rank, head_dim)."""
        return [(l.self_attn.nkv, l.self_attn.hd) for l in self.layers]

    def embed(self, input_ids):
        return ops.embedding(input_ids, self.embed_tokens, self.arch.embed_scale)

    def forward(self, batch, kv_caches, inputs_embeds=None):
        h = inputs_embeds if inputs_embeds is not None else self.embed(batch.input_ids)
        cs = self.cos_sin(h.device)
        if self._sequence_parallel_ok(h, batch):
            return self._forward_sequence_parallel(h, batch, kv_caches, cs)
        for i, layer in enumerate(self.layers):
            h = layer(h, batch, kv_caches[i], cs)
        return self.compute_logits(h, batch)

    # ------------------------------------------------------------------ sequence-parallel prefill
    def _sequence_parallel_ok(self, h, batch) -> bool:
        """Tensor-parallel prefill of a large batch on GPUs with the fused collectives: the residual
        stream is then kept sharded by token rows between the attention and MLP blocks."""
        if batch.is_decode or not h.is_cuda or batch.lora_mapping is not None:
            return False
        st = pstate.get_state()
        from ..parallel.fused_ops import fused_prefill_ok
        if (st.tp_size <= 1 or st.comm_backend != "fused" or st.symm is None or not st.sequence_parallel_ok
                or not fused_prefill_ok(st.tp_size)):
            return False
        if h.shape[0] < self.sp_min_tokens:
            return False
        l0 = self.layers[0]
        lin = (l0.self_attn.qkv_proj, l0.self_attn.o_proj, l0.mlp.gate_up_proj, l0.mlp.down_proj)
        if any(m.bias is not None for m in lin):
            return False
        # 16-bit layers or int4 layers (the int4 GEMM carries the same all-gather producer and
        # reduce-scatter epilogue); other quantised formats keep the replicated-activation prefill
        from ..layers.quantization.awq import Int4LinearMethod
        if any(m.quant_method is not None and not isinstance(m.quant_method, Int4LinearMethod) for m in lin):
            return False
        # int4 layers: opt-in.  Their all-gather producer pulls every token tile from its owner once per
        # weight tile (no staged copy yet): measured on 2 GPUs with the 9B int4 model, p50 time to first
        # token 647 ms sequence-parallel against 340 ms with replicated activations and GEMM->all-reduce.
        if any(m.quant_method is not None for m in lin) and not self.sp_int4:
            return False
        w = st.tp_size
        rpr = (h.shape[0] + w * 128 - 1) // (w * 128) * 128
        elem = h.element_size()
        return rpr * h.shape[1] * elem <= st.symm.xbuf_bytes and st.symm.fits_recv(rpr, h.shape[1], elem)

    def _forward_sequence_parallel(self, h_full, batch, kv_caches, cs):
        """One prefill forward with the hidden states sharded by token rows over the TP ranks:

            norm(shard) -> all-gather->GEMM (qkv, all tokens x local heads) -> rotary + cache + attention
            -> GEMM->reduce-scatter (+ residual shard) -> norm(shard) -> all-gather->GEMM (gate|up, gated)
            -> GEMM->reduce-scatter (+ residual shard)

        so every collective of the layer is fused into the GEMM next to it and the norms, residual adds
        and the staging copies touch 1/world of the tokens.  Tokens are padded to world x 128 rows."""
        from ..parallel import fused_ops
        st = pstate.get_state()
        w, r = st.tp_size, pstate.tp_rank()
        T, H = h_full.shape
        rpr = (T + w * 128 - 1) // (w * 128) * 128
        Tpad = rpr * w
        dev, dt = h_full.device, h_full.dtype
        h = torch.zeros(rpr, H, dtype=dt, device=dev)                 # this rank's rows of the residual stream
        lo, hi = r * rpr, min((r + 1) * rpr, T)
        if hi > lo:
            h[: hi - lo].copy_(h_full[lo:hi])
        l0 = self.layers[0].self_attn
        attn = torch.zeros(Tpad, l0.nh * l0.hd, dtype=dt, device=dev)  # rows beyond T stay zero
        cfg = batch.config
        for i, layer in enumerate(self.layers):
            at, mlp = layer.self_attn, layer.mlp
            x = layer.input_layernorm(h)
            qkv = fused_ops.allgather_gemm(x, at.qkv_proj, Tpad, rpr)[:T]
            k_cache, v_cache = kv_caches[i]
            ops.rope_and_cache(qkv, batch.positions, cs, batch.slot_mapping, k_cache, v_cache, at.nh, at.nkv, at.hd,
                               at.rot_dim, q_norm_w=at.q_norm.weight if at.qk_norm else None,
                               k_norm_w=at.k_norm.weight if at.qk_norm else None,
                               qk_norm_mode=(at.q_norm.w_mode if at.qk_norm else -1), eps=at.eps,
                               k_scale=cfg.k_scale, v_scale=cfg.v_scale)
            ops.paged_attention_prefill(qkv, k_cache, v_cache, batch.block_tables, batch.seq_lens, batch.cu_q,
                                        batch.max_q_len, at.nh, at.nkv, at.hd, at.sm_scale, at.window, 0.0,
                                        cfg.k_scale, cfg.v_scale, out=attn[:T])
            fused_ops.gemm_reduce_scatter(attn, at.o_proj, h, rpr, out_shard=h)
            x = layer.post_attention_layernorm(h)
            a = fused_ops.allgather_gemm(x, mlp.gate_up_proj, Tpad, rpr, gated_act=mlp.gate_up_proj.gated_act)
            fused_ops.gemm_reduce_scatter(a, mlp.down_proj, h, rpr, out_shard=h)
        full = pstate.all_gather_rows(h)[:T]
        return self.compute_logits(full, batch)

    def compute_logits(self, h, batch):
        last = h if batch.logits_indices is None else h.index_select(0, batch.logits_indices)
        x = self.norm(last)
        if self.tie:
            logits = ops.linear(x, self.embed_tokens, out_dtype=torch.float32)
        else:
            logits = self.lm_head(x, out_dtype=torch.float32)
            if self.lm_head.tp > 1:
                greedy_out = batch.extras.get("greedy_out") if batch.extras else None
                st = pstate.get_state()
                if (greedy_out is not None and logits.is_cuda and st.comm_backend == "fused" and st.symm is not None
                        and st.argmax_ok and logits.shape[0] <= 1024):
                    # only the greedy tokens are wanted: agree on them from the vocabulary slices (one kernel,
                    # 16 bytes per row and peer) instead of gathering [rows, vocab] logits
                    from ..parallel import fused_ops
                    fused_ops.argmax_vocab_parallel(logits, pstate.tp_rank() * logits.shape[1], out=greedy_out)
                    batch.extras["greedy_done"] = True
                    return logits
                logits = pstate.all_gather_last_dim(logits)
        return logits

    # ------------------------------------------------------------------ loading
    def load_weights(self, weights):
        """weights: iterable of (hf_name, tensor).  Returns the set of consumed names."""
        from ..loaders.weight_utils import load_llama_style
        loaded = load_llama_style(self, weights)
        if self.fuse_rmsnorm:
            for layer in self.layers:
                layer.fold_norms()
        return loaded
