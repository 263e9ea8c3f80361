"""Row-parallel GEMM + all-reduce micro-benchmark across ranks (one process per GPU, launched with torchrun):

  python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m deepseek_v4_2080ti_b200.utils.tp_microbench \\
      --rows 8192 --out-features 5120 --in-features 17408

For every variant the time is CUDA-event time on each rank, max over ranks, median of the iterations:
  gemm        this rank's K-shard GEMM alone (no communication)
  nccl        GEMM, then NCCL all-reduce of the bf16 output (the baseline)
  oneshot     GEMM whose epilogue pushes each partial tile to every peer and sums (peer stores over NVLink)
  twoshot     GEMM whose epilogue sends partials to the tile owner, which reduces and returns the tile
  rs          sequence-parallel form: GEMM whose epilogue pushes each partial tile to the owner of its token rows
  rs_gather   rs, then the owners' reduce + residual + RMSNorm + all-gather kernel, then the wait for every peer's rows
  sp_sublayer rs -> reduce/norm/gather -> the next column-parallel GEMM consuming the gathered rows tile by tile
              (``--next-features`` outputs per rank); ar_sublayer is the same work as GEMM + NCCL all-reduce ->
              add + norm on all rows -> GEMM
Roofline per call = max(FLOPs / measured bf16 GEMM peak, bytes this rank must send / NVLink bandwidth per direction).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


# Device-side delay queued before the first event of every timed iteration (about 0.5 ms): the launches of the
# measured function are already in the queue when the delay ends, so the interval between the events holds kernel
# time and dependencies, not the host's launch latency (tens of microseconds per launch, comparable to the kernels).
HEAD_START_CYCLES = 1_000_000


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", dest="t", type=int, default=8192)
    ap.add_argument("--out-features", dest="n", type=int, default=5120)
    ap.add_argument("--in-features", dest="k", type=int, default=17408, help="full K; every rank holds K / world")
    ap.add_argument("--next-features", dest="n2", type=int, default=0, help="per-rank width of the column-parallel GEMM "
                    "that follows (default: 2 * in-features / world, a gate_up shard)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--gemm-peak-tflops", type=float, default=1397.7)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    a = ap.parse_args()
    from ..formats import fp8 as fp8fmt
    from ..ops import _lib, gemm
    from ..parallel import tp
    rank, world, local = tp.init_distributed()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = tp.PeerComm(slot_elems=a.t * a.n)
    ks = a.k // world
    torch.manual_seed(rank)
    w = torch.randn(a.n, ks, device=dev) * 0.02
    q, s = fp8fmt.quantize_block128(w)
    pl = gemm.PackedLinear.from_fp8(q, s)
    del w
    x = torch.randn(a.t, ks, device=dev).bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        ts = []
        for i in range(a.iters + 3):
            flush.zero_()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(HEAD_START_CYCLES)      # the host queues fn() while the device is still busy here
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= 3:
                ts.append(e0.elapsed_time(e1))
        ts.sort()
        t = torch.tensor([ts[len(ts) // 2]], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    out = {}
    out["gemm"] = timed(lambda: gemm.linear(x, pl, stream=False))
    out["nccl"] = timed(lambda: dist.all_reduce(gemm.linear(x, pl, stream=False)))
    out["oneshot"] = timed(lambda: comm.linear_allreduce(x, pl, two_shot=False))
    out["twoshot"] = timed(lambda: comm.linear_allreduce(x, pl, two_shot=True))
    # ---- sequence-parallel forms
    from ..ops import basic
    rows = comm.sp_rows(a.t, a.n)
    n2 = a.n2 or 2 * ks
    if rows:
        w2 = gemm.PackedLinear.from_bf16((torch.randn(n2, a.n, device=dev) * 0.02).bfloat16())
        gamma = torch.zeros(a.n, device=dev, dtype=torch.bfloat16)
        h_shard = torch.randn(rows, a.n, device=dev).bfloat16()
        h_full = torch.randn(a.t, a.n, device=dev).bfloat16()
        y2 = torch.empty(a.t, n2, device=dev, dtype=torch.bfloat16)

        def rs_gather():
            comm.linear_rs(x, pl)
            comm.reduce_norm_gather(h_shard, gamma, 1e-6, True)
            comm.wait_gather(rows)

        def sp_sublayer():
            comm.linear_rs(x, pl)
            comm.linear_ag(comm.reduce_norm_gather(h_shard, gamma, 1e-6, True), w2, out=y2)

        def ar_sublayer():
            d = gemm.linear(x, pl, stream=False)
            dist.all_reduce(d)
            gemm.linear(basic.add_rmsnorm(h_full, d, gamma, 1e-6, True), w2, out=y2)

        def rs_only():
            # the push alone cannot be repeated without its consumer (the flags and slots belong to one epoch pair),
            # so the consumer runs outside the events
            comm.linear_rs(x, pl)

        ts = []
        for i in range(a.iters + 3):
            flush.zero_()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(HEAD_START_CYCLES)
            e0.record()
            rs_only()
            e1.record()
            comm.reduce_norm_gather(h_shard, None, 1e-6, True, gather=False)
            torch.cuda.synchronize()
            if i >= 3:
                ts.append(e0.elapsed_time(e1))
        ts.sort()
        tt = torch.tensor([ts[len(ts) // 2]], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        out["rs"] = float(tt.item())
        out["rs_gather"] = timed(rs_gather)
        out["sp_sublayer"] = timed(sp_sublayer)
        out["ar_sublayer"] = timed(ar_sublayer)
        out["gemm2"] = timed(lambda: gemm.linear(h_full, w2, out=y2))
    comm.check()
    flops = 2.0 * a.t * a.n * ks
    payload = a.t * a.n * 2
    sent = {"oneshot": (world - 1) * payload, "twoshot": 2 * (world - 1) / world * payload,
            "nccl": 2 * (world - 1) / world * payload}
    if rank == 0:
        rec = {"op": "gemm_allreduce", "world": world, "t": a.t, "n": a.n, "k_per_rank": ks, "ms": out}
        for v in ("nccl", "oneshot", "twoshot"):
            roof = max(flops / (a.gemm_peak_tflops * 1e9), sent[v] / (a.link_gbs * 1e6))
            rec[f"{v}_roofline_ms"] = round(roof, 4)
            rec[f"{v}_fraction_of_roofline"] = round(roof / out[v], 3)
        if "rs" in out:
            one_way = (world - 1) / world * payload / (a.link_gbs * 1e6)        # ms to send (or receive) one shard set
            g1 = flops / (a.gemm_peak_tflops * 1e9)
            g2 = 2.0 * a.t * n2 * a.n / (a.gemm_peak_tflops * 1e9)
            rec["next_features_per_rank"] = n2
            rec["rs_roofline_ms"] = round(max(g1, one_way), 4)
            rec["rs_fraction_of_roofline"] = round(max(g1, one_way) / out["rs"], 3)
            # reduce-scatter and all-gather each move (W-1)/W of the tensor; the first can hide under GEMM 1, the second
            # under GEMM 2, so the bound of the whole sub-layer is the slower of the math and the two transfers
            sub = max(g1 + g2, 2 * one_way)
            rec["sp_sublayer_roofline_ms"] = round(sub, 4)
            rec["sp_sublayer_fraction_of_roofline"] = round(sub / out["sp_sublayer"], 3)
            rec["ar_sublayer_fraction_of_roofline"] = round(sub / out["ar_sublayer"], 3)
        print(json.dumps(rec), flush=True)
    comm.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
