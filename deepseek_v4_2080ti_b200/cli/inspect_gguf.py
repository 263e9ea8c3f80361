"""Inspect a GGUF checkpoint: metadata, tensor inventory by type, family detection, validation against the family's
tensor naming, runtime capability per tensor type and the placement plan for a GPU box.
(Reference: src/cli/inspect_gguf.py; cpp_engine/tools/inspect_gguf.cpp.)"""
from __future__ import annotations

import argparse
import json
import sys

from ..formats.gguf import read_bundle
from ..models import registry


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="inspect_gguf")
    ap.add_argument("path")
    ap.add_argument("--tensors", action="store_true", help="list every tensor")
    ap.add_argument("--grep", default="")
    ap.add_argument("--validate", action="store_true")
    ap.add_argument("--placement", action="store_true")
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--gpu-memory-gib", type=float, default=180.0)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    b = read_bundle(a.path)
    out = {"architecture": b.architecture, "files": len(b.files), "tensors": len(b.tensors),
           "metadata": {k: (v if not isinstance(v, (list, tuple)) or len(v) <= 8 else f"<{len(v)} items>")
                        for k, v in b.metadata.items()}}
    by_type: dict[str, int] = {}
    for ti in b.tensors.values():
        by_type[ti.ggml_type.name] = by_type.get(ti.ggml_type.name, 0) + ti.nbytes
    out["bytes_by_type"] = by_type
    out["capability"] = {t: registry.capability_status(b.tensors[next(n for n, x in b.tensors.items() if x.ggml_type.name == t)].ggml_type)[0]
                         for t in by_type}
    if a.tensors:
        out["tensor_list"] = [{"name": n, "type": ti.ggml_type.name, "shape": list(ti.shape), "bytes": ti.nbytes}
                              for n, ti in b.tensors.items() if a.grep in n]
    rc = 0
    if a.validate or a.placement:
        spec = registry.detect(b)
        rep = spec.validate(b)
        out["family"] = spec.display_name
        out["validation"] = {"ok": rep.ok, "missing": rep.missing[:20], "unexpected": rep.unexpected[:20],
                             "unsupported": dict(list(rep.unsupported.items())[:20]), "total_bytes": rep.total_bytes,
                             "routed_bytes": rep.routed_bytes}
        rc = 0 if rep.ok else 1
        if a.placement:
            hw = registry.HardwareProfile(a.gpus, a.gpu_memory_gib, f"{a.gpus}x{a.gpu_memory_gib:g}GiB")
            out["placement"] = [vars(d) for d in spec.placement(rep, hw)]
    if a.json:
        print(json.dumps(out, default=str))
    else:
        for k, v in out.items():
            print(f"{k}: {json.dumps(v, default=str)}")
    return rc


if __name__ == "__main__":
    sys.exit(main())
