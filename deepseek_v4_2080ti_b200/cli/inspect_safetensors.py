"""Inspect a safetensors checkpoint directory without loading it: shards, tensors (dtype, shape, bytes), totals per
dtype, an optional name filter, and for Qwen-style hybrid checkpoints the weight-map coverage audit (missing /
unexpected tensors, shapes, dtypes, tensor-parallel divisibility; FP8 block-128 and mixed NVFP4 matrices).

    python -m deepseek_v4_2080ti_b200.cli.inspect_safetensors CKPT_DIR [--grep STR] [--audit] [--tp-world N] [--json]

The native executable offers the same through ``--inspect`` / ``--qwen-audit``
(reference: cpp_engine/engine/main.cpp inspection modes, cpp_engine/tools/qwen_audit.cpp)."""
from __future__ import annotations

import argparse
import json
import os
import sys


def scan(directory: str) -> dict:
    from ..formats.safetensors_io import SafetensorsFile
    shards = sorted(f for f in os.listdir(directory) if f.endswith(".safetensors"))
    if not shards:
        raise FileNotFoundError(f"no .safetensors shard in {directory}")
    tensors, by_dtype = [], {}
    for fn in shards:
        f = SafetensorsFile(os.path.join(directory, fn))
        for name, info in f.header.items():
            b, e = info["data_offsets"]
            tensors.append({"name": name, "dtype": info["dtype"], "shape": list(info["shape"]), "bytes": e - b, "shard": fn})
            by_dtype[info["dtype"]] = by_dtype.get(info["dtype"], 0) + (e - b)
    index = os.path.join(directory, "model.safetensors.index.json")
    indexed = None
    if os.path.exists(index):
        wm = json.load(open(index)).get("weight_map", {})
        have = {t["name"]: t["shard"] for t in tensors}
        indexed = {"entries": len(wm), "missing_from_shards": sorted(n for n in wm if n not in have)[:20],
                   "wrong_shard": sorted(n for n, s in wm.items() if n in have and have[n] != s)[:20]}
    return {"directory": directory, "shards": shards, "tensors": tensors, "bytes_by_dtype": by_dtype,
            "total_bytes": sum(by_dtype.values()), "index": indexed}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="inspect_safetensors")
    ap.add_argument("checkpoint")
    ap.add_argument("--grep", default="", help="only tensors whose name contains this")
    ap.add_argument("--audit", action="store_true", help="check the Qwen-style weight map (needs config.json)")
    ap.add_argument("--tp-world", type=int, default=1)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    rep = scan(a.checkpoint)
    shown = [t for t in rep["tensors"] if a.grep in t["name"]]
    audit = None
    if a.audit:
        from .. import pocketllm_cpp as core
        audit = dict(core.qwen_audit(a.checkpoint, a.tp_world))
    if a.json:
        print(json.dumps({**{k: v for k, v in rep.items() if k != "tensors"}, "tensors": shown, "audit": audit}))
    else:
        for t in shown:
            print(f"{t['name']} {t['dtype']} {t['shape']} {t['bytes']} {t['shard']}")
        print(f"shards={len(rep['shards'])} tensors={len(shown)}/{len(rep['tensors'])} total_bytes={rep['total_bytes']} "
              + " ".join(f"{k}={v}" for k, v in sorted(rep["bytes_by_dtype"].items())))
        if rep["index"] is not None:
            print(f"index entries={rep['index']['entries']} missing_from_shards={len(rep['index']['missing_from_shards'])} "
                  f"wrong_shard={len(rep['index']['wrong_shard'])}")
        if audit is not None:
            for key in ("missing", "unexpected", "wrong_shape", "wrong_dtype", "not_divisible"):
                for n in audit[key]:
                    print(f"audit_{key}={n}")
            print(f"audit ok={int(audit['ok'])} expected={audit['expected']} found={audit['found']} tp_world={a.tp_world}")
    return 0 if audit is None or audit["ok"] else 3


if __name__ == "__main__":
    sys.exit(main())
