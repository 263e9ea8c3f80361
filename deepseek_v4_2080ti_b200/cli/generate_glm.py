"""Greedy generation from a GLM-style (``glm-dsa``) GGUF checkpoint: the family-agnostic GGUF driver under the name the
reference gives its GLM entry point (src/cli/generate_glm.py); the family is detected from the file's metadata.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m deepseek_v4_2080ti_b200.cli.generate_glm \\
        --gguf glm.gguf --token-ids 1,2,3 --max-new-tokens 64"""
from __future__ import annotations

import sys

from .generate_gguf import main

if __name__ == "__main__":
    sys.exit(main())
