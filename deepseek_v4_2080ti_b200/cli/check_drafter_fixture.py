"""Check the DFlash2 drafter statement stage by stage against an exported fixture, or export one.

A fixture is a tensor file (``formats/tensor_file.py``) holding ``target_taps`` [rows, n_taps * hidden] for the context
rows at ``position_offset ..``, the anchor token, and - in a full fixture - every named intermediate stage of one
proposal.  The reference exports such fixtures from the upstream PyTorch drafter and compares its device runtime with
them (cpp_engine/tests/export_qwen_dflash2_fixture.py, compare_qwen_dflash2_parity.py); this tool does the same for
``models/qwen_dflash2_ref.py``:

    python -m deepseek_v4_2080ti_b200.cli.check_drafter_fixture --drafter DRAFTER_DIR --target TARGET_DIR \\
        --fixture capture_or_fixture.qdf2 [--export out.qdf2] [--viterbi] [--rtol 3e-2] [--cosine 0.999] [--strict-tokens]

``TARGET_DIR`` supplies ``model.language_model.embed_tokens.weight`` and ``lm_head.weight``.  With ``--export`` the
stages computed here are written out (the capture's taps included).  Stages present in the fixture are compared in
the order they were produced: floating stages pass when ``max |a - b| <= rtol * max |b| + atol`` and the cosine is at
least ``--cosine``; integer stages (tokens, candidates, the selected path) are counted, and fail the check only with
``--strict-tokens``, since near-ties may flip under fp16 rounding.  Exit status 0 when every compared stage passes.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def find_tensor(directory: str, name: str) -> torch.Tensor:
    """One tensor of a (possibly sharded) safetensors checkpoint, without reading the rest."""
    import os

    from ..formats.safetensors_io import SafetensorsFile
    index = os.path.join(directory, "model.safetensors.index.json")
    shards = None
    if os.path.exists(index):
        shard = json.load(open(index)).get("weight_map", {}).get(name)
        shards = [shard] if shard else None
    for fn in shards or sorted(f for f in os.listdir(directory) if f.endswith(".safetensors")):
        f = SafetensorsFile(os.path.join(directory, fn))
        if name in f.keys():
            return f.get(name)
    raise KeyError(f"{name} not found in {directory}")


def run_stages(drafter_dir: str, embedding: torch.Tensor, head: torch.Tensor, taps: torch.Tensor, position_offset: int,
               anchor: int, viterbi: bool = False) -> dict[str, torch.Tensor]:
    from ..models import qwen_dflash2_ref as df
    cfg, w = df.load_dflash2(drafter_dir)
    dr = df.QwenDFlash2Ref(cfg, w, embedding, head, max_context=position_offset + taps.shape[0] + cfg.block_size,
                           viterbi=viterbi)
    stages: dict[str, torch.Tensor] = {"target_taps": taps.clone()}
    dr.debug = lambda name, t: stages.setdefault(name, t.detach().clone())
    dr.reset(position_offset)
    dr.append_target_taps(taps, position_offset)
    dr.propose(anchor)
    return stages


def compare(got: dict[str, torch.Tensor], want: dict[str, torch.Tensor], rtol: float, atol: float, cosine: float,
            strict_tokens: bool) -> tuple[list[dict], bool]:
    rows, ok = [], True
    for name, a in got.items():
        if name not in want:
            continue
        b = want[name]
        row = {"stage": name, "shape": list(a.shape)}
        if a.numel() != b.numel():
            row.update(status="FAIL", why=f"{list(a.shape)} here, {list(b.shape)} in the fixture")
            ok = False
        elif not b.is_floating_point():
            diff = int((a.reshape(-1).long() != b.reshape(-1).long()).sum())
            row.update(mismatches=diff, of=b.numel(), status="ok" if diff == 0 else ("FAIL" if strict_tokens else "differs"))
            ok = ok and (diff == 0 or not strict_tokens)
        else:
            x, y = a.reshape(-1).double(), b.reshape(-1).double()
            err, ref = float((x - y).abs().max()), float(y.abs().max())
            den = float(x.norm() * y.norm())
            cos = float(x @ y) / den if den > 0 else float(torch.equal(x, y))
            good = err <= rtol * ref + atol and cos >= cosine
            row.update(max_abs_err=err, max_abs_ref=ref, cosine=cos, status="ok" if good else "FAIL")
            ok = ok and good
        rows.append(row)
    return rows, ok


def main(argv=None) -> int:
    from ..formats import tensor_file as tf
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--drafter", required=True)
    ap.add_argument("--target", required=True)
    ap.add_argument("--fixture", required=True)
    ap.add_argument("--export", default="")
    ap.add_argument("--viterbi", action="store_true")
    ap.add_argument("--rtol", type=float, default=3e-2)
    ap.add_argument("--atol", type=float, default=1e-3)
    ap.add_argument("--cosine", type=float, default=0.999)
    ap.add_argument("--strict-tokens", action="store_true")
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    fx = tf.read(args.fixture)
    if "target_taps" not in fx.tensors:
        print("the fixture holds no target_taps", file=sys.stderr)
        return 2
    emb = find_tensor(args.target, "model.language_model.embed_tokens.weight")
    head = find_tensor(args.target, "lm_head.weight")
    stages = run_stages(args.drafter, emb, head, fx.tensors["target_taps"].float(), fx.position_offset, fx.anchor_token,
                        args.viterbi)
    if args.export:
        n = tf.write(args.export, tf.TensorFile(fx.position_offset, fx.anchor_token, stages))
        print(f"wrote {len(stages)} stages, {n} bytes: {args.export}", file=sys.stderr)
    rows, ok = compare(stages, {k: v for k, v in fx.tensors.items() if k != "target_taps"}, args.rtol, args.atol,
                       args.cosine, args.strict_tokens)
    if args.json:
        print(json.dumps({"ok": ok, "compared": len(rows), "stages": rows}))
    else:
        for r in rows:
            if "cosine" in r:
                print(f"{r['status']:8s} {r['stage']:40s} max|err| {r['max_abs_err']:.3e} of {r['max_abs_ref']:.3e}  cos {r['cosine']:.6f}")
            elif "mismatches" in r:
                print(f"{r['status']:8s} {r['stage']:40s} {r['mismatches']} of {r['of']} differ")
            else:
                print(f"{r['status']:8s} {r['stage']:40s} {r['why']}")
        first = next((r["stage"] for r in rows if r["status"] == "FAIL"), None)
        print(f"{len(rows)} stages compared: " + ("all within tolerance" if ok else f"first failure at {first}"))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
