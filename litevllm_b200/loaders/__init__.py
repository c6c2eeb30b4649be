"""Model and tokenizer loading.

``get_model`` builds the model class for the configured architecture directly on the target device
and streams weights into it from safetensors shards (dense, AWQ, compressed-tensors), a GGUF file,
or the synthetic random-init stream.  Reference: vllm/model_executor/model_loader/__init__.py:
943-1085 (``get_model``) and :912-940 (``get_tokenizer``).
"""
from __future__ import annotations

import json
from collections.abc import Iterator
from pathlib import Path

import torch

from ..logger import init_logger
from ..models.registry import ModelRegistry

logger = init_logger(__name__)


def resolve_device(device: str = "auto") -> torch.device:
    if device in (None, "auto"):
        if torch.cuda.is_available():
            return torch.device("cuda", torch.cuda.current_device())
        return torch.device("cpu")
    return torch.device(device)


def iter_safetensors(model_dir: str | Path) -> Iterator[tuple[str, torch.Tensor]]:
    """Yield every tensor of every ``*.safetensors`` shard (index order when an index exists)."""
    from safetensors import safe_open
    d = Path(model_dir)
    index = d / "model.safetensors.index.json"
    if index.is_file():
        files = sorted(set(json.loads(index.read_text())["weight_map"].values()))
    else:
        files = sorted(p.name for p in d.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors files under {d}")
    for fname in files:
        with safe_open(str(d / fname), framework="pt", device="cpu") as f:
            for key in f.keys():
                yield key, f.get_tensor(key)


def synthetic_weights(vllm_config, device) -> Iterator[tuple[str, torch.Tensor]]:
    from . import synth
    mc = vllm_config.model_config
    fam = mc.arch.family
    # small models draw on the CPU (bit-identical across devices and ranks); big ones on the device
    big = mc.arch.hidden_size * mc.arch.num_layers >= 4096 * 30
    gen_dev = str(device) if (big and device.type == "cuda") else "cpu"
    if fam in ("llama", "qwen2", "qwen2_vl"):
        return synth.iter_llama_weights(mc.arch, mc.seed, torch.float32 if not big else mc.dtype, gen_dev)
    if fam == "gemma4":
        return synth.iter_gemma4_weights(mc.arch, mc.seed, mc.dtype, gen_dev)
    if fam == "deepseek_mla":
        return synth.iter_deepseek_weights(mc.arch, mc.seed, mc.dtype, gen_dev)
    if fam == "qwen3_5":
        return synth.iter_qwen35_weights(mc.arch, mc.seed, mc.dtype, gen_dev)
    if fam == "deepseek_v4_flash":
        return iter(())             # the model draws its own seeded weights when no tensor arrives
    raise ValueError(f"no synthetic weight stream for family {fam}")


def get_model(vllm_config, device: str | torch.device = "auto") -> torch.nn.Module:
    mc = vllm_config.model_config
    dev = resolve_device(device if isinstance(device, str) else str(device))
    cls = ModelRegistry.resolve_model_cls(mc.arch.architecture, mc.arch.family)
    with torch.device(dev):
        model = cls(vllm_config)
    if mc.synthetic:
        weights = synthetic_weights(vllm_config, dev)
    elif mc.is_gguf:
        from .gguf import iter_gguf_weights
        weights = iter_gguf_weights(mc.model, mc.arch)
    else:
        weights = iter_safetensors(mc.model)
    # repacked int4 layouts from an earlier start of the same checkpoint on the same rank layout
    cache_path = None
    if not mc.synthetic and not mc.is_gguf and dev.type == "cuda":
        from . import repack_cache
        from ..parallel import state as pstate
        st = pstate.get_state()
        cache_path = repack_cache.cache_file(mc.model, st.rank, max(st.world_size, 1), mc.dtype)
        if cache_path is not None and repack_cache.attach(model, cache_path, dev):
            logger.info("int4 layouts attached from %s; packed tensors of the checkpoint are not read", cache_path)
            weights = repack_cache.lazy_safetensors_without_packed(mc.model)
            cache_path = None
    consumed = model.load_weights(weights)
    if cache_path is not None:
        n = repack_cache.save(model, cache_path)
        if n:
            logger.info("wrote the repacked layouts of %d int4 layers to %s", n, cache_path)
    logger.info("loaded %d tensors into %s on %s", len(consumed), cls.__name__, dev)
    model.eval()
    return model


class DummyTokenizer:
    """Stand-in when no tokenizer files exist (synthetic models, token-id prompts)."""
    eos_token_id = None
    bos_token_id = None
    pad_token_id = 0
    chat_template = None

    def __init__(self, vocab_size: int = 32000):
        self.vocab_size = vocab_size

    def encode(self, text: str, add_special_tokens: bool = True) -> list[int]:
        return [ord(c) % self.vocab_size for c in text]

    def decode(self, ids, skip_special_tokens: bool = True, **_) -> str:
        return " ".join(str(int(i)) for i in ids)

    def __call__(self, text, **kw):
        return {"input_ids": self.encode(text)}

    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True, **_):
        text = "".join(f"<{m['role']}>{m['content']}\n" for m in messages)
        if add_generation_prompt:
            text += "<assistant>"
        return self.encode(text) if tokenize else text

    def __len__(self):
        return self.vocab_size


def get_tokenizer(path: str, trust_remote_code: bool = False, revision: str | None = None,
                  vocab_size: int = 32000):
    p = Path(path)
    has_files = p.is_dir() and any((p / f).exists() for f in ("tokenizer.json", "tokenizer.model", "tokenizer_config.json"))
    if not has_files:
        return DummyTokenizer(vocab_size)
    from transformers import AutoTokenizer
    try:
        return AutoTokenizer.from_pretrained(str(p), trust_remote_code=trust_remote_code, revision=revision)
    except Exception as e:  # slow-tokenizer fallback
        logger.warning("fast tokenizer failed (%s); trying the slow one", e)
        try:
            return AutoTokenizer.from_pretrained(str(p), use_fast=False, trust_remote_code=trust_remote_code)
        except Exception:
            return DummyTokenizer(vocab_size)
