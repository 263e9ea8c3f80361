"""``bench.py --impl reference``: run the unmodified reference (installed under ``baseline/_ref``)
through its own public API on the same metric/config, or report why it cannot run."""
from __future__ import annotations

import os

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def run(args) -> dict:
    if not os.path.isdir(os.path.join(REF, "pocketllm")):
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed (offline pip build of /root/reference did not complete)"}
    return {"impl": "reference",
            "unavailable": "the pip-installed reference has no Qwen3.5 runtime: its Qwen path needs the CMake-built pocketllm_cpp module (cpp_engine/), which setup.py does not build"}
