"""Helpers shared by the sampling stages (reference: vllm/engine/sampling/utils.py)."""
from __future__ import annotations


def collect_eos_ids(tokenizer, hf_eos_ids, sampling_params) -> frozenset[int]:
    """EOS set of a request = tokenizer EOS + model-config EOS + ``stop_token_ids``."""
    ids: set[int] = set()
    tok_eos = getattr(tokenizer, "eos_token_id", None)
    if isinstance(tok_eos, int):
        ids.add(tok_eos)
    elif isinstance(tok_eos, (list, tuple)):
        ids.update(int(t) for t in tok_eos)
    ids.update(int(t) for t in (hf_eos_ids or []))
    ids.update(int(t) for t in (sampling_params.stop_token_ids or []))
    return frozenset(ids)


def is_greedy(sp) -> bool:
    return sp.temperature <= 1e-6
