"""Tokenizer access: protocol, cached Hugging Face loading, a small registry and incremental
detokenisation.  Reference: vllm/tokenizers/{hf,protocol,registry,detokenizer_utils}.py."""
from .detokenizer_utils import IncrementalDetokenizer, detokenize_incrementally
from .hf import get_cached_tokenizer
from .protocol import TokenizerLike
from .registry import TokenizerRegistry, get_tokenizer

__all__ = ["IncrementalDetokenizer", "detokenize_incrementally", "get_cached_tokenizer", "TokenizerLike",
           "TokenizerRegistry", "get_tokenizer"]
