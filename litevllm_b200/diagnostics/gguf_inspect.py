"""What a GGUF file holds, read from its header alone (no tensor payload is touched).

    python -m litevllm_b200.diagnostics.gguf_inspect model.gguf [--json] [--tensors PATTERN] [--metadata]

Prints the architecture and the configuration this engine derives from the file, bytes and tensor counts per
block format, the stacked expert tensors (experts x rows x columns, format, bytes per expert: what a staging
budget has to hold per slot), per-layer byte totals, and tensors whose format this engine cannot run.
Same role as tests/tools/deepseek_v4_flash_inspect.py and inspect_deepseek_v4_flash_expert_shapes.py of the
reference.
"""
from __future__ import annotations

import argparse
import json
import re
import sys
from collections import defaultdict


def inspect(path: str, pattern: str | None = None) -> dict:
    from ..loaders.gguf import _NP, BLOCK, TYPE_NAMES, GGUFFile, hf_config_from_gguf
    g = GGUFFile(path)
    by_type: dict[str, dict] = defaultdict(lambda: {"tensors": 0, "bytes": 0, "elements": 0})
    per_layer: dict[int, int] = defaultdict(int)
    experts, unsupported, listed = [], [], []
    rx = re.compile(pattern) if pattern else None
    total = 0
    for name, t in g.tensors.items():
        ty, shape, nbytes = t["type"], t["shape"], t["nbytes"]
        tname = TYPE_NAMES.get(ty, f"type{ty}")
        n = 1
        for d in shape:
            n *= d
        row = by_type[tname]
        row["tensors"] += 1
        row["bytes"] += nbytes
        row["elements"] += n
        total += nbytes
        m = re.match(r"blk\.(\d+)\.", name)
        if m:
            per_layer[int(m.group(1))] += nbytes
        if ty not in _NP and ty != 30 and ty not in BLOCK:
            unsupported.append({"name": name, "type": tname})
        if len(shape) == 3 and "_exps" in name:
            experts.append({"name": name, "experts": shape[0], "rows": shape[1], "columns": shape[2], "type": tname,
                            "bytes_per_expert": nbytes // max(1, shape[0])})
        if rx is not None and rx.search(name):
            listed.append({"name": name, "shape": list(shape), "type": tname, "bytes": nbytes, "offset": t["offset"]})
    for row in by_type.values():
        row["bits_per_weight"] = round(8.0 * row["bytes"] / max(1, row["elements"]), 3)
    try:
        derived = hf_config_from_gguf(path)
        config_error = None
    except Exception as e:          # noqa: BLE001 - an inspection tool reports what it cannot derive
        derived, config_error = None, f"{type(e).__name__}: {e}"
    per_block = defaultdict(int)
    for e in experts:
        m = re.match(r"blk\.(\d+)\.", e["name"])
        per_block[int(m.group(1)) if m else -1] += e["bytes_per_expert"]
    return {"path": str(path), "architecture": g.arch(), "alignment": g.alignment, "tensors": len(g.tensors),
            "bytes": total, "by_type": dict(sorted(by_type.items(), key=lambda kv: -kv[1]["bytes"])),
            "layers": len(per_layer), "bytes_per_layer_max": max(per_layer.values(), default=0),
            "expert_tensors": experts, "expert_bytes_per_slot_per_block": max(per_block.values(), default=0),
            "expert_bytes_total": sum(e["bytes_per_expert"] * e["experts"] for e in experts),
            "unsupported": unsupported, "derived_config": derived, "config_error": config_error,
            "metadata": g.metadata, "listed": listed}


def slots_for_budget(info: dict, budget_gb: float) -> dict:
    """What a staging budget of ``budget_gb`` buys: slots per MoE block and the share of the experts they hold."""
    blocks = len({re.match(r"blk\.(\d+)\.", e["name"]).group(1) for e in info["expert_tensors"]
                  if re.match(r"blk\.(\d+)\.", e["name"])}) or 1
    per_slot = info["expert_bytes_per_slot_per_block"]
    experts = max((e["experts"] for e in info["expert_tensors"]), default=0)
    if not per_slot or not experts:
        return {"blocks": 0, "slots_per_block": 0, "experts_per_block": 0, "resident_share": 1.0}
    slots = min(experts, int(budget_gb * 2 ** 30 // blocks // per_slot))
    return {"blocks": blocks, "slots_per_block": slots, "experts_per_block": experts,
            "resident_share": round(slots / experts, 4)}


def render(info: dict, show_metadata: bool = False) -> str:
    gb = 2 ** 30
    out = [f"{info['path']}: architecture {info['architecture'] or '?'}, {info['tensors']} tensors, "
           f"{info['bytes'] / gb:.3f} GiB, alignment {info['alignment']}, {info['layers']} layers"]
    out.append(f"{'format':10s} {'tensors':>8s} {'GiB':>10s} {'bits/weight':>12s}")
    for name, row in info["by_type"].items():
        out.append(f"{name:10s} {row['tensors']:8d} {row['bytes'] / gb:10.3f} {row['bits_per_weight']:12.3f}")
    if info["expert_tensors"]:
        first = [e for e in info["expert_tensors"] if e["name"].startswith(info["expert_tensors"][0]["name"].split(".ffn")[0])]
        out.append(f"routed experts: {info['expert_bytes_total'] / gb:.3f} GiB in all; one slot of one block holds "
                   f"{info['expert_bytes_per_slot_per_block'] / 2 ** 20:.2f} MiB")
        for e in first:
            out.append(f"  {e['name']}: {e['experts']} x {e['rows']} x {e['columns']} {e['type']}, "
                       f"{e['bytes_per_expert'] / 2 ** 20:.2f} MiB per expert")
    if info["unsupported"]:
        out.append("formats this engine cannot run: " + ", ".join(sorted({u["type"] for u in info["unsupported"]}))
                   + f" ({len(info['unsupported'])} tensors, first: {info['unsupported'][0]['name']})")
    if info["config_error"]:
        out.append("no configuration derived: " + info["config_error"])
    elif info["derived_config"]:
        keys = ("architectures", "num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
                "vocab_size", "n_routed_experts", "num_experts_per_tok", "max_position_embeddings")
        out.append("derived: " + ", ".join(f"{k}={info['derived_config'][k]}" for k in keys if k in info["derived_config"]))
    for t in info["listed"]:
        out.append(f"  {t['name']}: {t['shape']} {t['type']} {t['bytes']} bytes at {t['offset']}")
    if show_metadata:
        for k, v in sorted(info["metadata"].items()):
            s = json.dumps(v, default=str)
            out.append(f"  {k} = {s if len(s) <= 120 else s[:117] + '...'}")
    return "\n".join(out)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("path")
    ap.add_argument("--json", action="store_true", help="print everything as one JSON object")
    ap.add_argument("--tensors", default=None, help="also list the tensors whose name matches this regular expression")
    ap.add_argument("--metadata", action="store_true", help="also print the metadata keys")
    ap.add_argument("--device-budget-gb", type=float, default=0.0,
                    help="also print how many expert slots per block this staging budget holds")
    a = ap.parse_args(argv)
    try:
        info = inspect(a.path, a.tensors)
    except (ValueError, OSError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    if a.device_budget_gb > 0:
        info["staging"] = slots_for_budget(info, a.device_budget_gb)
    print(json.dumps(info, default=str) if a.json else render(info, a.metadata))
    if a.device_budget_gb > 0 and not a.json:
        st = info["staging"]
        print(f"a budget of {a.device_budget_gb:g} GiB holds {st['slots_per_block']} of {st['experts_per_block']} experts "
              f"in each of {st['blocks']} blocks ({100 * st['resident_share']:.1f} % resident)")
    return 1 if info["unsupported"] or info["config_error"] else 0


if __name__ == "__main__":
    sys.exit(main())
