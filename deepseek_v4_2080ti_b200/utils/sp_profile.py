"""One-GPU driver for the sequence-parallel kernels: the ranks of a tensor-parallel group are emulated on one device
(``PeerComm.local_group``) and stepped phase by phase, so each kernel can be timed or captured by a profiler without a
multi-rank launch (every flag a kernel waits for was raised by a kernel that has already finished; "peer" stores land in
this GPU's own memory, so link time is NOT part of these numbers - they show the kernels' own cost).

  python -m deepseek_v4_2080ti_b200.utils.sp_profile --world 4 --rows 1024 --hidden 5120 --k 1024 --next 3072

Per phase: CUDA-event time of the launch of ONE emulated rank (median over ranks and iterations)."""
from __future__ import annotations

import argparse
import json

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=4)
    ap.add_argument("--rows", type=int, default=1024, help="token rows per rank")
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--k", type=int, default=1024, help="K of the row-parallel GEMM per rank")
    ap.add_argument("--next", dest="n2", type=int, default=3072, help="width of the column-parallel GEMM per rank")
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    from ..ops import _lib, gemm
    from ..parallel import tp

    t = a.world * a.rows
    comms = tp.PeerComm.local_group(a.world, slot_elems=t * a.hidden, budget_ms=500.0)
    assert comms[0].sp_rows(t, a.hidden) == a.rows
    dev = "cuda"
    xs = [torch.randn(t, a.k, device=dev).bfloat16() for _ in range(a.world)]
    w1 = gemm.PackedLinear.from_bf16((torch.randn(a.hidden, a.k, device=dev) * 0.02).bfloat16())
    w2 = gemm.PackedLinear.from_bf16((torch.randn(a.n2, a.hidden, device=dev) * 0.02).bfloat16())
    gamma = torch.zeros(a.hidden, device=dev, dtype=torch.bfloat16)
    shards = [torch.randn(a.rows, a.hidden, device=dev).bfloat16() for _ in range(a.world)]
    y2 = torch.empty(t, a.n2, device=dev, dtype=torch.bfloat16)
    times = {"rs_gemm": [], "reduce_norm_gather": [], "ag_gemm": []}

    def timed(key, fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(1_000_000)      # ~0.5 ms on the device: the launch below is queued before the first event fires
        e0.record()
        out = fn()
        e1.record()
        torch.cuda.synchronize()
        times[key].append(e0.elapsed_time(e1))
        return out

    for it in range(a.iters + 1):
        for r in range(a.world):
            timed("rs_gemm", lambda: comms[r].linear_rs(xs[r], w1))
        g = [timed("reduce_norm_gather", lambda: comms[r].reduce_norm_gather(shards[r], gamma, 1e-6, True))
             for r in range(a.world)]
        for r in range(a.world):
            timed("ag_gemm", lambda: comms[r].linear_ag(g[r], w2, out=y2))
        if it == 0:
            for v in times.values():
                v.clear()
    _lib.check_status()
    med = {k: round(sorted(v)[len(v) // 2], 4) for k, v in times.items()}
    part_bytes = a.world * a.rows * a.hidden * 2
    print(json.dumps({"world": a.world, "rows_per_rank": a.rows, "hidden": a.hidden, "k_per_rank": a.k, "next": a.n2,
                      "ms": med,
                      "reduce_norm_gather_bytes": {"partials_read": part_bytes, "residual_rw": 2 * a.rows * a.hidden * 2,
                                                   "rows_written": a.world * a.rows * a.hidden * 2},
                      "note": "one device, emulated ranks: peer stores are local"}), flush=True)
    for c in comms:
        c.close()


if __name__ == "__main__":
    main()
