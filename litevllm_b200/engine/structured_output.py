"""Structured-output constraints (filled in by the constraint implementations below).
``make_constraint_factory`` returns a callable building a per-request constraint object with the
interface ``apply_mask(logits_row)``, ``on_token(token_id)``, ``should_finish()``."""
from __future__ import annotations


def make_constraint_factory(tokenizer, vocab_size: int):
    def factory(params):
        from .structured_constraints import build_constraint
        return build_constraint(params, tokenizer, vocab_size)
    return factory
