"""Resident multi-sequence engine over stdin / stdout for the MLA + routed-expert family:

    python -m deepseek_v4_2080ti_b200.cli.resident_engine --model CKPT_DIR_OR_GGUF --max-slots 8 --max-context 8192

loads the checkpoint once (safetensors directory with a DeepSeek-style config.json, or a ``glm-dsa`` GGUF file) and
then answers one JSON command per line (``runtime/resident_engine.py``: alloc / prefill / decode / verify / free /
reset / stats / stop); a failing command is reported and the loop goes on.  Single rank.  Reference: the
``--persistent`` modes of cpp_engine/engine/main.cpp that keep a PersistentEngine alive between requests."""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--max-slots", type=int, default=4)
    ap.add_argument("--max-context", type=int, default=4096)
    ap.add_argument("--chunk", type=int, default=2048)
    a = ap.parse_args(argv)
    import torch

    from ..models import mla_moe_gpu as mg
    from ..ops import _lib
    from ..runtime.resident_engine import ResidentEngine
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if a.model.endswith(".gguf"):
        from ..formats.gguf import read_bundle
        from ..models import registry
        bundle = read_bundle(a.model)
        spec = registry.detect(bundle)
        _, rt = spec.build_runtime(bundle, dev, 0, 1, None, max_slots=max(2, a.max_slots), max_context=a.max_context)
        if not isinstance(rt, mg.MlaMoeBatchRuntime):
            raise SystemExit(f"{spec.architecture}: no resident multi-sequence runtime for this family")
    else:
        from ..formats import safetensors_io
        from ..models.mla_moe import MlaMoeConfig
        raw = json.load(open(os.path.join(a.model, "config.json")))
        if not MlaMoeConfig.is_mla_moe_json(raw):
            raise SystemExit("config.json does not describe an MLA + routed-expert checkpoint")
        cfg = MlaMoeConfig.from_json(raw)
        w = mg.MlaMoeGpuWeights(cfg, safetensors_io.read_checkpoint(a.model), dev,
                                dense_fp8=str(raw.get("dtype", "bf16")).lower() == "fp8")
        rt = mg.MlaMoeBatchRuntime(cfg, w, max_slots=a.max_slots, max_context=a.max_context)
    eng = ResidentEngine(rt, to_ids=lambda toks: torch.tensor(toks, dtype=torch.int32, device=dev), chunk=a.chunk)
    print(json.dumps({"ready": True, "max_slots": rt.max_slots, "max_context": rt.max_context, "pages": rt.free_pages()}), flush=True)
    eng.serve(sys.stdin, sys.stdout, after_command=_lib.check_status)
    return 0


if __name__ == "__main__":
    sys.exit(main())
