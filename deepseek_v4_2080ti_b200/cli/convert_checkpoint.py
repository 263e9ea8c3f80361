"""Re-encode the matrices of a safetensors checkpoint into another weight format, shard by shard:

    bf16 | fp8 (E4M3, 128x128 block scales, ``weight_scale_inv``) | fp4 (E2M1 + E8M0 per 32, ``scale``)
    | nvfp4 (E2M1 + E4M3 per 16 + fp32 global scale: ``weight_packed`` / ``weight_scale`` / ``weight_global_scale``)
    | int8 (symmetric, one fp32 ``scale`` per output row: the W8A8 layout of the host expert kernels)

The reference's converter turns FP4 / FP8 checkpoints into INT8 W8A8 because its GPUs have no FP8 or FP4 tensor path
(src/cli/convert_checkpoint.py, src/models/deepseek_v4/loader.py:36-45); on B200 those formats run natively, so the
useful directions are bf16 -> fp8 / fp4 and back; the INT8 target serves the host (CPU) expert path."""
from __future__ import annotations

import argparse
import json
import sys

import torch


def convert_tensor(name: str, w: torch.Tensor, scale: torch.Tensor | None, src: str, dst: str) -> dict[str, torch.Tensor]:
    from ..formats import fp4 as fp4fmt
    from ..formats import fp8 as fp8fmt
    from ..formats import nvfp4 as nvfmt
    base = name[:-len(".weight")]
    if src == "nvfp4":
        w = nvfmt.dequantize(w, scale[0], scale[1])
    elif src == "fp8":
        w = fp8fmt.dequantize_block128(w, scale.float())
    elif src == "fp4":
        w = fp4fmt.dequantize(w, scale)
    elif src == "int8":
        w = w.float() * scale.float()[:, None]
    w = w.float()
    if dst == "bf16":
        return {name: w.bfloat16()}
    if dst == "fp8":
        q, s = fp8fmt.quantize_block128(w)
        return {name: q, base + ".weight_scale_inv": s.bfloat16()}
    if dst == "fp4":
        q, s = fp4fmt.quantize(w)
        return {name: q, base + ".scale": s}
    if dst == "int8":
        sc = w.abs().amax(-1) / 127.0
        q = torch.where(sc[:, None] > 0, torch.round(w / sc.clamp_min(1e-30)[:, None]).clamp(-127, 127), torch.zeros_like(w))
        return {name: q.to(torch.int8), base + ".scale": sc.float()}
    if dst == "nvfp4":
        q, s, g = nvfmt.quantize(w)
        return {base + ".weight_packed": q, base + ".weight_scale": s, base + ".weight_global_scale": g}
    raise ValueError(dst)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="convert_checkpoint")
    ap.add_argument("src_dir")
    ap.add_argument("dst_dir")
    ap.add_argument("--to", choices=["bf16", "fp8", "fp4", "nvfp4", "int8"], required=True)
    ap.add_argument("--match", default="", help="only matrices whose name contains this (others are copied)")
    ap.add_argument("--min-dim", type=int, default=128, help="leave smaller matrices alone")
    a = ap.parse_args(argv)
    from ..formats import safetensors_io as sio
    state = dict(sio.read_checkpoint(a.src_dir))
    out: dict[str, torch.Tensor] = {}
    converted = 0
    for name, w in state.items():
        if name.endswith((".weight_scale_inv", ".scale", ".weight_scale", ".weight_global_scale")):
            continue
        if name.endswith(".weight_packed"):                         # an NVFP4 matrix: three tensors under one base name
            base = name[:-len(".weight_packed")]
            parts = (state[base + ".weight_scale"], state[base + ".weight_global_scale"])
            if a.to == "nvfp4" or a.match not in name:
                out[name], out[base + ".weight_scale"], out[base + ".weight_global_scale"] = w, *parts
            else:
                out.update(convert_tensor(base + ".weight", w, parts, "nvfp4", a.to))
                converted += 1
            continue
        base = name[:-len(".weight")] if name.endswith(".weight") else None
        sc_fp8 = state.get(base + ".weight_scale_inv") if base else None
        sc_fp4 = state.get(base + ".scale") if base else None
        src = "fp8" if sc_fp8 is not None else "bf16" if sc_fp4 is None else "int8" if w.dtype == torch.int8 else "fp4"
        ok = base is not None and w.dim() == 2 and a.match in name and \
            (a.to != "nvfp4" or w.shape[1] % 16 == 0) and \
            (src != "bf16" or (min(w.shape) >= a.min_dim and w.shape[1] % 128 == 0 and w.dtype in (torch.bfloat16, torch.float16, torch.float32)))
        if not ok or src == a.to:
            out[name] = w
            if sc_fp8 is not None:
                out[base + ".weight_scale_inv"] = sc_fp8
            if sc_fp4 is not None:
                out[base + ".scale"] = sc_fp4
            continue
        out.update(convert_tensor(name, w, sc_fp8 if sc_fp8 is not None else sc_fp4, src, a.to))
        converted += 1
    import os
    cfg = os.path.join(a.src_dir, "config.json")
    sio.write_checkpoint(a.dst_dir, iter(out.items()), config_json=open(cfg).read() if os.path.exists(cfg) else None)
    print(json.dumps({"tensors": len(out), "converted": converted, "to": a.to}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
