"""One eager decode step (or, with ``--prefill T``, one prefill of T tokens) of the 27B-shaped hybrid model between
cudaProfilerStart/Stop, for a per-kernel launch list:

  ncu --profile-from-start off --metrics gpu__time_duration.sum --clock-control none --csv \\
      --log-file launches.csv python -m deepseek_v4_2080ti_b200.utils.decode_profile --batch 1 --layers 8

Without ncu it prints the CUDA-event time of the step (eager launches, so launch gaps are included)."""
from __future__ import annotations

import argparse
import json

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--context", type=int, default=512)
    ap.add_argument("--prefill", type=int, default=0, help="profile one prefill of this many tokens instead of a decode step")
    ap.add_argument("--phases", choices=["off", "range", "timed"], default="off",
                    help="per-site phase profile of the prefill: NVTX ranges, or device-timed accumulators printed at the end")
    a = ap.parse_args()
    from ..models import qwen_hybrid as qh
    from .phase_profile import PROFILER
    from ..ops import _lib
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = qh.QwenHybridConfig(num_hidden_layers=a.layers)
    w = qh.QwenHybridWeights(cfg, qh.synth_state(cfg, 0, dev), dev)
    rt = qh.QwenHybridRuntime(cfg, w, max_slots=a.batch, max_context=a.context + 64)
    gen = torch.Generator().manual_seed(1)
    if a.prefill:
        rt = qh.QwenHybridRuntime(cfg, w, max_slots=2, max_context=a.prefill + 64)
        p = torch.randint(0, cfg.vocab_size, (a.prefill,), generator=gen, dtype=torch.int32).to(dev)
        s = rt.allocate()
        rt.prefill(s, p)
        rt.free(s)
        torch.cuda.synchronize()
        s = rt.allocate()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        PROFILER.set_mode(a.phases)
        torch.cuda.cudart().cudaProfilerStart()
        e0.record()
        rt.prefill(s, p)
        e1.record()
        torch.cuda.synchronize()
        torch.cuda.cudart().cudaProfilerStop()
        _lib.check_status()
        print(json.dumps({"prefill": a.prefill, "layers": a.layers, "ms": e0.elapsed_time(e1), "launches": rt.launches}))
        if a.phases == "timed":
            print(PROFILER.format())
        PROFILER.set_mode("off")
        return
    slots, cur = [], []
    for _ in range(a.batch):
        s = rt.allocate()
        p = torch.randint(0, cfg.vocab_size, (a.context,), generator=gen, dtype=torch.int32).to(dev)
        cur.append(rt.prefill(s, p))
        slots.append(s)
    tok = torch.cat(cur).to(torch.int32)
    for _ in range(2):
        tok = rt.decode(slots, tok, use_graph=False).to(torch.int32)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.cudart().cudaProfilerStart()
    e0.record()
    tok = rt.decode(slots, tok, use_graph=False).to(torch.int32)
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    _lib.check_status()
    print(json.dumps({"batch": a.batch, "layers": a.layers, "eager_step_ms": e0.elapsed_time(e1), "launches": rt.launches}))


if __name__ == "__main__":
    main()
