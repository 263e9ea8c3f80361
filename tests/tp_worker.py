"""Rank program for the multi-GPU tests (launched by torch.distributed.run from test_tp_multi_gpu.py).

Checks, on every rank: the peer-memory one-shot all-reduce and arg-max merge against NCCL, the GEMM with
the all-reduce fused into its epilogue against GEMM + NCCL all-reduce, and that a tensor-parallel tiny
model generates the same greedy tokens as the single-rank model.  Prints ``TP_WORKER_OK`` on success."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from deepseek_v4_2080ti_b200.formats import fp8 as fp8fmt  # noqa: E402
from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh  # noqa: E402
from deepseek_v4_2080ti_b200.ops import _lib, gemm  # noqa: E402
from deepseek_v4_2080ti_b200.parallel import tp  # noqa: E402


def main() -> None:
    rank, world, local = tp.init_distributed()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = tp.PeerComm(slot_elems=1 << 20)
    nccl = tp.TPComm()

    # one-shot all-reduce, several sizes, repeated (epochs advance, parity alternates)
    for it, n in enumerate([8, 5120, 5120, 40960, 1 << 20, 3 * 5120 + 8]):
        torch.manual_seed(100 + it * 8 + rank)
        a = torch.randn(n, device=dev).bfloat16()
        want = a.float().clone()
        dist.all_reduce(want)
        got = comm.all_reduce(a.clone())
        torch.cuda.synchronize()
        comm.check()
        err = (got.float() - want).abs().max() / want.abs().max()
        assert err < 2e-2, ("allreduce", n, err.item())
        # every rank holds the same bits
        ref = got.clone()
        dist.broadcast(ref, 0)
        assert torch.equal(ref, got), ("allreduce not identical across ranks", n)

    # arg-max merge
    torch.manual_seed(7 + rank)
    val = torch.randn(33, device=dev)
    idx = torch.randint(0, 1000, (33,), device=dev, dtype=torch.int32) + rank * 1000
    got = comm.argmax_merge(idx, val)
    want = nccl.argmax_merge(idx, val)
    torch.cuda.synchronize()
    comm.check()
    assert torch.equal(got.cpu(), want.cpu())

    # row-parallel GEMM with the all-reduce in the epilogue
    for t, n, kfull in [(1, 256, 1024), (48, 640, 2048), (300, 512, 1024), (130, 1024, 512)]:
        torch.manual_seed(5)                      # same full problem on every rank
        w = torch.randn(n, kfull, device=dev) * 0.05
        x = torch.randn(t, kfull, device=dev).bfloat16()
        r = torch.randn(t, n, device=dev).bfloat16()
        ks = kfull // world
        q, s = fp8fmt.quantize_block128(w[:, rank * ks:(rank + 1) * ks].contiguous())
        pl = gemm.PackedLinear.from_fp8(q, s)
        xs = x[:, rank * ks:(rank + 1) * ks].contiguous()
        part = gemm.linear(xs, pl, stream=False).float()
        dist.all_reduce(part)
        want = part + r.float()
        for two_shot in (False, True):
            got = comm.linear_allreduce(xs, pl, residual=r, two_shot=two_shot).clone()
            got2 = comm.linear_allreduce(xs, pl, residual=r, two_shot=two_shot).clone()
            torch.cuda.synchronize()
            comm.check()
            err = (got.float() - want).abs().max() / want.abs().max()
            assert err < 2e-2, ("gemm_allreduce", two_shot, t, n, kfull, err.item())
            assert torch.equal(got, got2)
            ref = got.clone()
            dist.broadcast(ref, 0)
            assert torch.equal(ref, got), ("fused all-reduce not identical across ranks", two_shot, t, n)

    # tensor-parallel model == single-rank model (greedy tokens)
    cfg = qh.QwenHybridConfig.tiny(layers=4)
    cfg = qh.QwenHybridConfig(vocab_size=512, hidden_size=256, intermediate_size=256 * world, num_hidden_layers=4,
                              num_attention_heads=2 * world, num_key_value_heads=world, linear_num_key_heads=world,
                              linear_num_value_heads=2 * world, max_position_embeddings=4096, full_attention_interval=2)
    state = list(qh.synth_state(cfg, 0, dev, std=0.05))
    torch.manual_seed(3)
    prompt = torch.randint(0, cfg.vocab_size, (150,), dtype=torch.int32)
    w1 = qh.QwenHybridWeights(cfg, iter(state), dev)
    single = qh.QwenHybridRuntime(cfg, w1, max_slots=1, max_context=512).generate(prompt, 10)
    del w1
    wt = qh.QwenHybridWeights(cfg, iter(state), dev, rank, world)
    for c, name in ((nccl, "nccl"), (comm, "peer")):
        rt = qh.QwenHybridRuntime(cfg, wt, max_slots=1, max_context=512, comm=c)
        out = rt.generate(prompt, 10)
        torch.cuda.synchronize()
        comm.check()
        agree = sum(a == b for a, b in zip(out, single))
        assert out[0] == single[0] and agree >= 8, (name, out, single)
        ref = torch.tensor(out, device=dev)
        dist.broadcast(ref, 0)
        assert ref.tolist() == out, ("ranks disagree", name)
    assert comm.fused_calls > 0
    comm.close()
    dist.barrier()
    if rank == 0:
        print("TP_WORKER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
