"""Sum importance-matrix GGUF files (one per rank or run) into one.  (Reference: src/cli/merge_imatrix.py.)"""
from __future__ import annotations

import argparse
import json
import sys

from ..formats.gguf.imatrix import merge_imatrix_files


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="merge_imatrix")
    ap.add_argument("inputs", nargs="+")
    ap.add_argument("-o", "--output", required=True)
    ap.add_argument("--dataset", default="runtime_capture_merged")
    ap.add_argument("--chunk-size", type=int, default=None)
    a = ap.parse_args(argv)
    print(json.dumps(merge_imatrix_files(a.inputs, a.output, a.dataset, a.chunk_size)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
