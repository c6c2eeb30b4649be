"""LRU prefix cache keyed by (namespace, token ids): cloned KV blocks of whole-block prompt prefixes
plus, for exact hits, the logits of the last prompt position.  Lookup returns the longest cached
prefix of the new prompt.  Entries count against a byte budget.  Disabled when capacity is 0.
Reference: vllm/engine/prefix_cache.py:10-124."""
from __future__ import annotations

import hashlib
from collections import OrderedDict
from dataclasses import dataclass


@dataclass
class PrefixEntry:
    tokens: tuple
    num_tokens: int
    blocks: list          # per layer (k, v) clones
    logits: object | None
    nbytes: int


def _namespace(st) -> str:
    mm = st.multi_modal_data
    if not mm:
        ns = ""
    else:
        h = hashlib.sha1()
        for k in sorted(mm):
            h.update(repr((k, mm[k] if isinstance(mm[k], (str, int)) else str(type(mm[k])))).encode())
            if isinstance(mm[k], (list, tuple)):
                for item in mm[k]:
                    h.update(str(item)[:256].encode())
        ns = h.hexdigest()
    lora = getattr(st.lora_request, "lora_name", "") if st.lora_request is not None else ""
    return f"{ns}|{lora}"


class PrefixCache:
    def __init__(self, max_entries: int = 0, max_bytes: int = 1 << 30):
        self.max_entries = max(0, int(max_entries))
        self.max_bytes = int(max_bytes)
        self._entries: OrderedDict[tuple, PrefixEntry] = OrderedDict()
        self._by_first: dict[tuple, set] = {}
        self.bytes_used = 0
        self.hits = self.misses = self.stores = self.evictions = 0

    @property
    def enabled(self) -> bool:
        return self.max_entries > 0

    def _key(self, st, n: int) -> tuple:
        return (_namespace(st), *st.prompt_token_ids[:n])

    def contains(self, st, n: int) -> bool:
        return self._key(st, n) in self._entries

    def lookup(self, st) -> PrefixEntry | None:
        if not self.enabled:
            return None
        ns = _namespace(st)
        ids = st.prompt_token_ids
        best = None
        for key in self._by_first.get((ns, ids[0]), ()):
            e = self._entries[key]
            if e.num_tokens <= len(ids) and (best is None or e.num_tokens > best.num_tokens):
                if tuple(ids[: e.num_tokens]) == e.tokens:
                    best = e
        if best is None:
            self.misses += 1
            return None
        self.hits += 1
        self._entries.move_to_end((ns, *best.tokens))
        return best

    def store(self, st, n: int, blocks, logits=None) -> None:
        if not self.enabled:
            return
        nbytes = sum(k.numel() * k.element_size() + v.numel() * v.element_size() for k, v in blocks)
        if logits is not None:
            nbytes += logits.numel() * logits.element_size()
        if nbytes > self.max_bytes:
            return
        key = self._key(st, n)
        self._drop(key)
        e = PrefixEntry(tuple(st.prompt_token_ids[:n]), n, blocks, logits, nbytes)
        self._entries[key] = e
        self._by_first.setdefault((key[0], key[1]), set()).add(key)
        self.bytes_used += nbytes
        self.stores += 1
        while len(self._entries) > self.max_entries or self.bytes_used > self.max_bytes:
            old_key = next(iter(self._entries))
            self._drop(old_key)
            self.evictions += 1

    def _drop(self, key) -> None:
        e = self._entries.pop(key, None)
        if e is None:
            return
        self.bytes_used -= e.nbytes
        s = self._by_first.get((key[0], key[1]))
        if s is not None:
            s.discard(key)
            if not s:
                del self._by_first[(key[0], key[1])]

    def clear(self) -> None:
        self._entries.clear()
        self._by_first.clear()
        self.bytes_used = 0

    def stats(self) -> dict:
        return {"enabled": self.enabled, "entries": len(self._entries), "bytes": self.bytes_used,
                "hits": self.hits, "misses": self.misses, "stores": self.stores, "evictions": self.evictions}
