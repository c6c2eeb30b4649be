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


def _content_digest(h, value) -> None:
    """Feed the full content of one multimodal value into ``h``.  Two requests may share a cache entry
    only if their images are byte-identical: a type name, a ``repr`` (which holds a memory address) or
    the first bytes of a data URL (JPEG headers and quantisation tables repeat) do not identify an image."""
    if value is None or isinstance(value, (bool, int, float)):
        h.update(repr(value).encode())
    elif isinstance(value, str):
        h.update(b"s")
        h.update(value.encode("utf-8", "surrogatepass"))
    elif isinstance(value, (bytes, bytearray, memoryview)):
        h.update(b"b")
        h.update(bytes(value))
    elif isinstance(value, (list, tuple)):
        h.update(f"l{len(value)}".encode())
        for item in value:
            _content_digest(h, item)
    elif isinstance(value, dict):
        h.update(f"d{len(value)}".encode())
        for k in sorted(value, key=str):
            h.update(str(k).encode())
            _content_digest(h, value[k])
    elif hasattr(value, "tobytes") and hasattr(value, "size") and hasattr(value, "mode"):   # PIL image
        h.update(f"pil{value.size}{value.mode}".encode())
        h.update(value.tobytes())
    elif hasattr(value, "detach") and hasattr(value, "cpu"):                                   # torch tensor
        import torch
        t = value.detach().cpu().contiguous()
        h.update(f"t{tuple(t.shape)}{t.dtype}".encode())
        h.update(t.reshape(-1).view(torch.uint8).numpy().tobytes())
    elif hasattr(value, "tobytes") and hasattr(value, "shape"):                                # numpy array
        h.update(f"n{tuple(value.shape)}{getattr(value, 'dtype', '')}".encode())
        h.update(value.tobytes())
    else:
        raise TypeError(f"cannot identify multimodal content of type {type(value).__name__}")


def _namespace(st) -> str | None:
    """Cache namespace of a request: digest of its multimodal content plus its LoRA name.  ``None``
    means the content could not be identified and the request must bypass the cache."""
    mm = st.multi_modal_data
    if not mm:
        ns = ""
    else:
        ns = getattr(st, "_mm_digest", False)      # hashed once per request: images can be megabytes
        if ns is False:
            h = hashlib.sha1()
            try:
                _content_digest(h, mm)
                ns = h.hexdigest()
            except Exception:
                ns = None
            try:
                st._mm_digest = ns
            except AttributeError:
                pass
        if ns is None:
            return None
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
        key = self._key(st, n)
        return key[0] is None or key in self._entries      # unidentifiable content: never stored, so report "present"

    def lookup(self, st) -> PrefixEntry | None:
        if not self.enabled:
            return None
        ns = _namespace(st)
        if ns is None:
            self.misses += 1
            return None
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
        if key[0] is None:
            return
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
