"""On-disk cache of repacked int4 weight layouts.

Loading an AWQ / compressed-tensors checkpoint reads every packed tensor, unpacks the nibbles, merges
the pieces of fused layers (q|k|v, gate|up), shards them for this rank and re-packs them into the layout
the tcgen05 int4 GEMM reads.  The result depends only on the checkpoint files, the rank layout and the
compute dtype, so it is written once to ``FASTINFERENCE_REPACK_CACHE_DIR`` and the next start of the same
model on the same layout attaches it and skips the packed tensors of the checkpoint altogether.

One file per (checkpoint fingerprint, rank, world size, dtype): a dict ``layer prefix -> {qw, scales_t,
zeros_t, N, K, group}`` saved with ``torch.save`` (written to a temporary name, then renamed).  The
fingerprint hashes the names, sizes and modification times of ``config.json`` and the weight shards, so a
changed checkpoint never meets a stale cache.  The reference persists only a tile-profile JSON
(vllm/kernels/triton/awq_fused_profile.json); it repacks on every start.
"""
from __future__ import annotations

import hashlib
import os
from pathlib import Path

import torch

_PACKED_SUFFIXES = ("qweight", "scales", "qzeros", "weight_packed", "weight_scale", "weight_zero", "weight_zero_point",
                    "weight_shape")


def cache_dir() -> Path | None:
    d = os.environ.get("FASTINFERENCE_REPACK_CACHE_DIR")
    return Path(d) if d else None


def fingerprint(model_dir: str | Path) -> str:
    d = Path(model_dir)
    h = hashlib.sha1()
    files = sorted([p for p in d.glob("*.safetensors")] + [p for p in (d / "config.json",) if p.is_file()])
    for p in files:
        st = p.stat()
        h.update(f"{p.name}:{st.st_size}:{st.st_mtime_ns};".encode())
    return h.hexdigest()[:20]


def cache_file(model_dir, rank: int, world: int, dtype: torch.dtype) -> Path | None:
    d = cache_dir()
    if d is None:
        return None
    return d / f"{fingerprint(model_dir)}-r{rank}of{world}-{str(dtype).replace('torch.', '')}.pt"


def _int4_layers(model) -> dict:
    out = {}
    for mod in model.modules():
        qm = getattr(mod, "quant_method", None)
        if qm is not None and hasattr(mod, "int4") and getattr(mod, "prefix", ""):
            out[mod.prefix] = mod
    return out


def save(model, path: Path) -> int:
    """Write the runtime layouts of every int4 layer of ``model``; returns how many layers were written."""
    entries = {}
    for prefix, mod in _int4_layers(model).items():
        w = mod.int4
        if w is None or w.qw is None:
            continue
        entries[prefix] = {"qw": w.qw.cpu(), "scales_t": w.scales_t.cpu(),
                           "zeros_t": None if w.zeros_t is None else w.zeros_t.cpu(),
                           "N": w.N, "K": w.K, "group": w.group}
    if not entries:
        return 0
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(f".tmp{os.getpid()}")
    torch.save(entries, tmp)
    os.replace(tmp, path)
    return len(entries)


def attach(model, path: Path, device) -> bool:
    """Give every int4 layer its cached runtime layout.  Returns True only when the cache covers every int4
    layer of the model with matching shapes (a partial or mismatching cache is ignored as a whole)."""
    from ..ops.awq import Int4Weight
    if not path.is_file():
        return False
    try:
        entries = torch.load(path, map_location="cpu", weights_only=True)
    except Exception:
        return False
    layers = _int4_layers(model)
    if not layers or set(layers) - set(entries):
        return False
    for prefix, mod in layers.items():
        e = entries[prefix]
        if (e["N"], e["K"]) != (mod.out_features, mod.in_features):
            return False
    for prefix, mod in layers.items():
        e = entries[prefix]
        mod.int4 = Int4Weight.from_runtime(e["qw"].to(device), e["scales_t"].to(device),
                                           None if e["zeros_t"] is None else e["zeros_t"].to(device),
                                           e["N"], e["K"], e["group"])
        mod._q_nib = mod._q_scales = mod._q_zeros = None
        mod._repack_cached = True
    return True


def skip_packed(weights):
    """Filter a checkpoint stream: drop the packed tensors (their layers came from the cache)."""
    for name, tensor in weights:
        if name.rpartition(".")[2] in _PACKED_SUFFIXES:
            continue
        yield name, tensor


def lazy_safetensors_without_packed(model_dir: str | Path):
    """Like ``iter_safetensors`` but never reads a packed tensor from disk."""
    import json

    from safetensors import safe_open
    d = Path(model_dir)
    index = d / "model.safetensors.index.json"
    if index.is_file():
        files = sorted(set(json.loads(index.read_text())["weight_map"].values()))
    else:
        files = sorted(p.name for p in d.glob("*.safetensors"))
    for fname in files:
        with safe_open(str(d / fname), framework="pt", device="cpu") as f:
            for key in f.keys():
                if key.rpartition(".")[2] in _PACKED_SUFFIXES:
                    continue
                yield key, f.get_tensor(key)
