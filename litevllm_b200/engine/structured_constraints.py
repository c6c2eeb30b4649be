"""Per-request structured-output constraints.

Preferred backend: xgrammar (JSON schema, ``json_object``, regex, EBNF grammar, ``choice`` compiled
as an alternation): each step fills a token bitmask for the request's row and masks the logits.
Fallbacks when xgrammar or a usable vocabulary is missing: a token-trie constraint for ``choice`` and
a prefix-validating JSON constraint that only lets through tokens keeping the text a valid JSON
prefix (checked over the most likely candidates).
Interface used by the sampler and output pipeline: ``apply_mask(logits_row)``, ``on_token(id)``,
``should_finish()``.  Reference: vllm/engine/structured_output_lite.py:18-398.
"""
from __future__ import annotations

import json
import re

import torch

from .errors import InvalidRequestError


def _vocab_strings(tokenizer, vocab_size: int) -> list[str] | None:
    get_vocab = getattr(tokenizer, "get_vocab", None)
    if get_vocab is None:
        return None
    vocab = get_vocab()
    out = [""] * max(vocab_size, (max(vocab.values()) + 1) if vocab else 0)
    for tok, idx in vocab.items():
        if 0 <= idx < len(out):
            out[idx] = tok
    return out


class XGrammarConstraint:
    _compilers: dict[int, tuple] = {}

    def __init__(self, params, tokenizer, vocab_size: int):
        import xgrammar as xgr
        key = id(tokenizer)
        entry = self._compilers.get(key)
        if entry is None:
            try:
                info = xgr.TokenizerInfo.from_huggingface(tokenizer, vocab_size=vocab_size)
            except Exception:
                vocab = _vocab_strings(tokenizer, vocab_size)
                if vocab is None:
                    raise
                info = xgr.TokenizerInfo(vocab, vocab_size=vocab_size)
            entry = (info, xgr.GrammarCompiler(info))
            self._compilers[key] = entry
        info, compiler = entry
        kind = params.kind()
        try:
            if kind == "json":
                schema = params.json if isinstance(params.json, str) else json.dumps(params.json)
                compiled = compiler.compile_json_schema(schema)
            elif kind == "json_object":
                compiled = compiler.compile_builtin_json_grammar()
            elif kind == "regex":
                compiled = compiler.compile_regex(params.regex)
            elif kind == "grammar":
                compiled = compiler.compile_grammar(params.grammar)
            elif kind == "choice":
                compiled = compiler.compile_regex("(" + "|".join(re.escape(c) for c in params.choice) + ")")
            else:
                raise InvalidRequestError(f"unsupported structured output kind {kind!r}")
        except InvalidRequestError:
            raise
        except Exception as e:
            raise InvalidRequestError(f"cannot compile structured output constraint: {e}") from None
        self.xgr = xgr
        self.matcher = xgr.GrammarMatcher(compiled)
        self.bitmask = xgr.allocate_token_bitmask(1, info.vocab_size)
        self.vocab_size = info.vocab_size

    def apply_mask(self, logits_row: torch.Tensor) -> None:
        self.matcher.fill_next_token_bitmask(self.bitmask, 0)
        row = logits_row[: self.vocab_size].unsqueeze(0)
        self.xgr.apply_token_bitmask_inplace(row, self.bitmask.to(row.device))
        if logits_row.shape[0] > self.vocab_size:
            logits_row[self.vocab_size:] = float("-inf")

    def on_token(self, token_id: int) -> None:
        if not self.matcher.is_terminated():
            self.matcher.accept_token(int(token_id))

    def should_finish(self) -> bool:
        return self.matcher.is_terminated()


class ChoiceTrieConstraint:
    """Token-level trie over the tokenisations of the allowed strings."""

    def __init__(self, choices: list[str], tokenizer, vocab_size: int):
        if not choices:
            raise InvalidRequestError("choice needs at least one option")
        self.root: dict = {}
        for c in choices:
            node = self.root
            for t in tokenizer.encode(c, add_special_tokens=False) if _takes_kw(tokenizer) else tokenizer.encode(c):
                node = node.setdefault(int(t), {})
            node[None] = True
        self.node = self.root
        self.done = False

    def apply_mask(self, logits_row: torch.Tensor) -> None:
        allowed = [t for t in self.node if t is not None]
        if not allowed:
            return
        keep = torch.tensor(allowed, dtype=torch.long, device=logits_row.device)
        vals = logits_row[keep].clone()
        logits_row.fill_(float("-inf"))
        logits_row[keep] = vals

    def on_token(self, token_id: int) -> None:
        self.node = self.node.get(int(token_id), {})
        if not [t for t in self.node if t is not None]:
            self.done = True

    def should_finish(self) -> bool:
        return self.done


def _takes_kw(tokenizer) -> bool:
    try:
        tokenizer.encode("a", add_special_tokens=False)
        return True
    except TypeError:
        return False


def _is_json_prefix(text: str) -> bool:
    """True when ``text`` can still be extended to a valid JSON document."""
    stack, in_str, esc = [], False, False
    for ch in text:
        if in_str:
            if esc:
                esc = False
            elif ch == "\\":
                esc = True
            elif ch == '"':
                in_str = False
            continue
        if ch == '"':
            in_str = True
        elif ch in "{[":
            stack.append(ch)
        elif ch in "}]":
            if not stack or (stack[-1] == "{") != (ch == "}"):
                return False
            stack.pop()
        elif not (ch.isalnum() or ch in " \t\n\r:,.-+eE"):
            return False
    return True


def _json_complete(text: str) -> bool:
    try:
        json.loads(text)
        return text.strip()[:1] in "{["
    except Exception:
        return False


class JsonPrefixConstraint:
    """Keeps the decoded text a valid JSON prefix; inspects the ``top_n`` most likely tokens."""

    def __init__(self, tokenizer, top_n: int = 256):
        self.tokenizer, self.top_n = tokenizer, top_n
        self.ids: list[int] = []
        self.done = False

    def _text(self, ids) -> str:
        return self.tokenizer.decode(ids)

    def apply_mask(self, logits_row: torch.Tensor) -> None:
        k = min(self.top_n, logits_row.shape[0])
        cand = torch.topk(logits_row, k).indices.tolist()
        base = self._text(self.ids)
        ok = [t for t in cand if _is_json_prefix(self._text(self.ids + [t])) and
              (base.strip() or self._text([t]).strip()[:1] in "{[ \n")]
        if not ok:
            return
        keep = torch.tensor(ok, dtype=torch.long, device=logits_row.device)
        vals = logits_row[keep].clone()
        logits_row.fill_(float("-inf"))
        logits_row[keep] = vals

    def on_token(self, token_id: int) -> None:
        self.ids.append(int(token_id))
        if _json_complete(self._text(self.ids)):
            self.done = True

    def should_finish(self) -> bool:
        return self.done


def build_constraint(params, tokenizer, vocab_size: int):
    kind = params.kind()
    if kind is None:
        return None
    if kind == "structural_tag":
        raise InvalidRequestError("structural_tag constraints are not supported")
    try:
        return XGrammarConstraint(params, tokenizer, vocab_size)
    except InvalidRequestError:
        raise
    except Exception:
        pass
    if kind == "choice":
        return ChoiceTrieConstraint(list(params.choice), tokenizer, vocab_size)
    if kind in ("json", "json_object"):
        return JsonPrefixConstraint(tokenizer)
    raise InvalidRequestError(f"structured output kind {kind!r} needs the xgrammar backend")
