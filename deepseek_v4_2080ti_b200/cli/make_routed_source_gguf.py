"""Copy the routed-expert tensors (``*_exps.weight``) of a checkpoint into a GGUF of their own, optionally only a range
of experts: the source file an expert-parallel rank maps.  (Reference: src/cli/make_routed_source_gguf.py.)"""
from __future__ import annotations

import argparse
import json
import sys

from ..formats.gguf import read_bundle, write_gguf


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="make_routed_source_gguf")
    ap.add_argument("path")
    ap.add_argument("-o", "--output", required=True)
    ap.add_argument("--experts", default="", help="lo:hi, half-open (default: all)")
    a = ap.parse_args(argv)
    b = read_bundle(a.path)
    lo, hi = (int(x) for x in a.experts.split(":")) if a.experts else (0, None)
    tensors, kept = [], 0
    for name, ti in b.tensors.items():
        if not name.endswith("_exps.weight") or len(ti.shape) != 3:
            continue
        raw = b.raw(name)
        h = ti.shape[0] if hi is None else min(hi, ti.shape[0])
        tensors.append((name, raw[lo:h].contiguous(), ti.ggml_type, (h - lo, *ti.shape[1:])))
        kept += 1
    if not tensors:
        print("no routed-expert tensors found", file=sys.stderr)
        return 1
    meta = dict(b.metadata)
    meta["general.routed_source.expert_lo"] = lo
    meta["general.routed_source.expert_hi"] = -1 if hi is None else hi
    write_gguf(a.output, meta, tensors)
    print(json.dumps({"tensors": kept, "expert_lo": lo, "expert_hi": hi}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
