"""Child process of ``bench.py --impl reference``: drives the UNMODIFIED reference project (installed
under ``baseline/_ref``) through its own public API on one GPU and prints one JSON line.

Nothing from this repository's engine is imported here.  The reference loads models from a
checkpoint directory and tokenises string prompts, so this script first writes a synthetic
TinyLlama-shaped checkpoint (random N(0, 0.02) bf16 weights in safetensors + a word-level tokenizer
whose word ``w<i>`` is token id ``i``) to a temporary directory, then runs the same protocol as the
engine's own arm: submit B prompts, step until every admitted request has its first token (TTFT),
W warm-up steps, K timed steps bracketed by CUDA events, counting the tokens the steps return.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time
from pathlib import Path


def write_checkpoint(out: Path, cfg: dict, seed: int = 0) -> None:
    import torch
    from safetensors.torch import save_file
    out.mkdir(parents=True, exist_ok=True)
    (out / "config.json").write_text(json.dumps(cfg))
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    hd = H // cfg["num_attention_heads"]
    q, kv = cfg["num_attention_heads"] * hd, cfg["num_key_value_heads"] * hd
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    g = torch.Generator(device=dev).manual_seed(seed)

    def w(*shape):
        return (torch.randn(*shape, generator=g, device=dev) * 0.02).to(torch.bfloat16).cpu()
    t = {"model.embed_tokens.weight": w(V, H), "model.norm.weight": torch.ones(H, dtype=torch.bfloat16),
         "lm_head.weight": w(V, H)}
    for i in range(L):
        p = f"model.layers.{i}."
        t[p + "self_attn.q_proj.weight"] = w(q, H)
        t[p + "self_attn.k_proj.weight"] = w(kv, H)
        t[p + "self_attn.v_proj.weight"] = w(kv, H)
        t[p + "self_attn.o_proj.weight"] = w(H, q)
        t[p + "mlp.gate_proj.weight"] = w(I, H)
        t[p + "mlp.up_proj.weight"] = w(I, H)
        t[p + "mlp.down_proj.weight"] = w(H, I)
        t[p + "input_layernorm.weight"] = torch.ones(H, dtype=torch.bfloat16)
        t[p + "post_attention_layernorm.weight"] = torch.ones(H, dtype=torch.bfloat16)
    save_file(t, str(out / "model.safetensors"))
    # word-level tokenizer: "w17 w4" -> [17, 4]
    from tokenizers import Tokenizer, models, pre_tokenizers
    vocab = {f"w{i}": i for i in range(3, V)}
    vocab.update({"<u>": 0, "<b>": 1, "<e>": 2})
    tok = Tokenizer(models.WordLevel(vocab=vocab, unk_token="<u>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok.save(str(out / "tokenizer.json"))
    (out / "tokenizer_config.json").write_text(json.dumps(
        {"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "<e>", "bos_token": "<b>", "unk_token": "<u>",
         "pad_token": "<u>", "model_max_length": 1 << 20}))
    (out / "special_tokens_map.json").write_text(json.dumps(
        {"eos_token": "<e>", "bos_token": "<b>", "unk_token": "<u>", "pad_token": "<u>"}))


class CopyCounter:
    """Counts the bytes that cross the host/device boundary while ONE untimed engine step runs, by
    wrapping the torch entry points a Python engine can move data with (tensor construction on a CUDA
    device from host data, ``.to`` / ``.cuda`` / ``.cpu`` / ``copy_`` across devices, ``.item`` /
    ``.tolist`` / ``.numpy`` on CUDA tensors).  The reference's code is not touched; the wrappers are
    installed after the timed region and removed again."""

    def __init__(self, torch):
        self.torch = torch
        self.h2d = 0
        self.d2h = 0
        self._saved = []

    @staticmethod
    def _nbytes(t):
        return int(t.numel() * t.element_size())

    def _patch(self, owner, name, make):
        orig = getattr(owner, name)
        self._saved.append((owner, name, orig))
        setattr(owner, name, make(orig))

    def __enter__(self):
        torch, me = self.torch, self
        T = torch.Tensor

        def is_cuda_dev(d):
            return d is not None and str(d).startswith("cuda")

        def ctor(orig):
            def f(data, *a, **k):
                out = orig(data, *a, **k)
                if isinstance(out, T) and out.is_cuda and not (isinstance(data, T) and data.is_cuda):
                    me.h2d += me._nbytes(out)
                return out
            return f

        def mover(orig):
            def f(self_, *a, **k):
                out = orig(self_, *a, **k)
                if isinstance(out, T) and out is not self_:
                    if out.is_cuda and not self_.is_cuda:
                        me.h2d += me._nbytes(out)
                    elif self_.is_cuda and not out.is_cuda:
                        me.d2h += me._nbytes(self_)
                return out
            return f

        def copy_(orig):
            def f(self_, src, *a, **k):
                if isinstance(src, T):
                    if self_.is_cuda and not src.is_cuda:
                        me.h2d += me._nbytes(self_)
                    elif src.is_cuda and not self_.is_cuda:
                        me.d2h += me._nbytes(self_)
                return orig(self_, src, *a, **k)
            return f

        def reader(orig):
            def f(self_, *a, **k):
                if self_.is_cuda:
                    me.d2h += me._nbytes(self_)
                return orig(self_, *a, **k)
            return f

        for name in ("tensor", "as_tensor"):
            self._patch(torch, name, ctor)
        for name in ("to", "cuda", "cpu"):
            self._patch(T, name, mover)
        self._patch(T, "copy_", copy_)
        for name in ("item", "tolist", "numpy", "__int__", "__float__", "__bool__", "__index__"):
            self._patch(T, name, reader)
        return self

    def __exit__(self, *exc):
        for owner, name, orig in reversed(self._saved):
            setattr(owner, name, orig)
        self._saved = []
        return False


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-dir", required=True)
    ap.add_argument("--steps", type=int, required=True)
    ap.add_argument("--warmup", type=int, required=True)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--ckpt-dir", default="/tmp/fi_ref_ckpt_tinyllama")
    args = ap.parse_args()
    sys.path.insert(0, args.ref_dir)
    import torch
    B, P, K, W = args.batch, args.prompt_len, args.steps, args.warmup
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 2048,
           "num_hidden_layers": 22, "num_attention_heads": 32, "num_key_value_heads": 4,
           "intermediate_size": 5632, "vocab_size": 32000, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
           "max_position_embeddings": 4096, "hidden_act": "silu", "tie_word_embeddings": False,
           "torch_dtype": "bfloat16", "eos_token_id": 2, "bos_token_id": 1}
    ckpt = Path(args.ckpt_dir)
    if not (ckpt / "model.safetensors").exists():
        write_checkpoint(ckpt, cfg)

    import vllm  # the reference package from baseline/_ref
    assert str(Path(vllm.__file__).resolve()).startswith(str(Path(args.ref_dir).resolve())), vllm.__file__
    from vllm import LLM, SamplingParams
    slack = (B + 7) // 8 + 2
    max_len = (P + 1 + W + K + slack + 16 + 15) // 16 * 16
    llm = LLM(str(ckpt), dtype="bfloat16", max_num_seqs=B, max_model_len=max_len,
              max_num_batched_tokens=max(8192, B * P),
              fastinference_config={"profile": "throughput", "kv_type": "fp16"})
    eng = llm.engine
    g = torch.Generator().manual_seed(1234)
    ids = torch.randint(3, cfg["vocab_size"], (B, P), generator=g)
    prompts = [" ".join(f"w{int(t)}" for t in row) for row in ids]
    sp = SamplingParams(temperature=0.0, max_tokens=1 + W + K + slack, min_tokens=1 + W + K + slack,
                        ignore_eos=True)
    # warm the kernels (Triton JIT) on a short request
    eng.add_request("warm", prompts[0], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    while eng.active_request_count > 0:
        eng.step()
    torch.cuda.synchronize()

    cap = int(getattr(eng, "max_active_requests", B))
    n_sub = min(B, cap * 4)
    t0 = time.perf_counter()
    for i in range(n_sub):
        eng.add_request(f"r{i}", prompts[i], sp)
    ttft, seen = {}, set()
    n_admit = min(n_sub, cap)
    guard = 0
    while len(ttft) < n_admit and guard < 100000:
        outs = eng.step() or []
        now = time.perf_counter()
        for o in outs:
            if o.request_id not in ttft and o.outputs and len(o.outputs[0].token_ids) > 0:
                ttft[o.request_id] = now - t0
        guard += 1
    for _ in range(W):
        eng.step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    n_tok = 0
    for _ in range(K):
        outs = eng.step() or []
        n_tok += len(outs)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    # one more, untimed, step with the copy counter installed: bytes in and out per step of the stock loop
    h2d_bytes = d2h_bytes = None
    try:
        with CopyCounter(torch) as cc:
            eng.step()
            torch.cuda.synchronize()
        h2d_bytes, d2h_bytes = cc.h2d, cc.d2h
    except Exception as e:   # the count is a label, never a reason to lose the measurement
        print(f"copy counter failed: {e!r}", file=sys.stderr)
    res = {"impl": "reference", "value": round(n_tok / (ms / 1e3), 1), "unit": "tok/s", "n_gpus": 1, "steps": K,
           "warmup": W, "ms_per_step": round(ms / K, 4), "tokens_in_timed_region": n_tok,
           "active_requests_cap": cap, "ttft_p50_ms": round(statistics.median(ttft.values()) * 1e3, 2) if ttft else None,
           "dtype": "bf16", "data": "synthetic",
           "e2e": {"value": round(n_tok / (ms / 1e3), 1), "unit": "tok/s", "ms_per_step": round(ms / K, 4),
                   "api": "reference LiteEngine.add_request + LiteEngine.step (host token lists in, sampled ids out)",
                   "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                   "bytes_counted_by": "torch entry points wrapped during one extra untimed step"},
           "config": {"model": "tinyllama-1.1b (random init N(0,0.02))", "global_batch": B, "prompt_len": P,
                      "seq_len": P + 1 + W + K, "parallelism": "single GPU (the reference has no distributed layer)",
                      "profile": "throughput", "kv_type": "fp16",
                      "note": f"the reference admits at most {cap} requests at a time; tokens/s counts what the timed steps produced"}}
    print("REFJSON " + json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
