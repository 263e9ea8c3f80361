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


def teacher_forced(rt, prompt, forced):
    """Greedy predictions of ``rt`` when it is fed ``forced`` (another run's tokens) instead of its own: position i
    holds the token predicted after prompt + forced[:i].  Unlike free-running generation, one flipped near-tie does
    not change everything after it, so runs that differ only in reduction order can be compared token by token."""
    dev = rt.device
    slot = rt.allocate()
    try:
        preds = [int(rt.prefill(slot, prompt.to(dev, torch.int32)).item())]
        for t in forced[:-1]:
            preds.append(int(rt.decode([slot], torch.tensor([t], dtype=torch.int32, device=dev)).item()))
        return preds
    finally:
        rt.free(slot)


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

    # decode-size row-parallel projection: the weight-streaming GEMM with the one-shot all-reduce in its epilogue
    for t, n, kfull in [(1, 256, 1024), (1, 5120, 2048 * world), (8, 640, 1024), (32, 1024, 512 * world)]:
        torch.manual_seed(9)
        w = torch.randn(n, kfull, device=dev) * 0.05
        x = torch.randn(t, kfull, device=dev).bfloat16()
        r = torch.randn(t, n, device=dev).bfloat16()
        ks = kfull // world
        if ks % 128:
            continue
        q, s = fp8fmt.quantize_block128(w[:, rank * ks:(rank + 1) * ks].contiguous())
        pl = gemm.PackedLinear.from_fp8(q, s)
        xs = x[:, rank * ks:(rank + 1) * ks].contiguous()
        part = gemm.linear_stream(xs, pl).float()
        want = part.clone()
        dist.all_reduce(want)
        want += r.float()
        got = comm.stream_allreduce(xs, pl, residual=r).clone()
        got2 = comm.stream_allreduce(xs, pl, residual=r).clone()
        torch.cuda.synchronize()
        comm.check()
        err = (got.float() - want).abs().max() / want.abs().max()
        assert err < 2e-2, ("stream_allreduce", t, n, kfull, err.item())
        assert torch.equal(got, got2)
        ref = got.clone()
        dist.broadcast(ref, 0)
        assert torch.equal(ref, got), ("fused decode all-reduce not identical across ranks", t, n)

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
        out = teacher_forced(rt, prompt, single)
        torch.cuda.synchronize()
        comm.check()
        agree = sum(a == b for a, b in zip(out, single))
        assert out[0] == single[0] and agree >= 8, (name, out, single)
        ref = torch.tensor(out, device=dev)
        dist.broadcast(ref, 0)
        assert ref.tolist() == out, ("ranks disagree", name)
    assert comm.fused_calls > 0

    # sequence-parallel prefill (reduce-scatter GEMM -> reduce + norm + gather -> all-gather GEMM) against the
    # all-reduce form of the same chunk: same logits within bf16 noise, same greedy continuation
    t_sp = 256 * world
    assert comm.sp_rows(t_sp, cfg.hidden_size) == 256
    torch.manual_seed(11)
    sp_prompt = torch.randint(0, cfg.vocab_size, (t_sp,), dtype=torch.int32)
    rt = qh.QwenHybridRuntime(cfg, wt, max_slots=1, max_context=t_sp + 64, comm=comm)
    outs = {}
    for sp in (False, True, True):
        comm.sp_enabled = sp
        calls0 = comm.fused_calls
        toks = rt.generate(sp_prompt, 6, chunk=t_sp)
        torch.cuda.synchronize()
        comm.check()
        outs.setdefault(sp, []).append((toks, rt.last_logits.clone() if hasattr(rt, "last_logits") else None))
        if sp:
            # per layer: 2 reduce-scatter GEMMs, 2 gathers, 2 all-gather GEMMs; + the final gather
            assert comm.fused_calls - calls0 >= 6 * cfg.num_hidden_layers + 1, comm.fused_calls - calls0
    (ta, _), (tb, _), (tc, _) = outs[False][0], outs[True][0], outs[True][1]
    assert tb == tc, ("sequence-parallel prefill not reproducible", tb, tc)
    comm.sp_enabled = True
    tf = teacher_forced(rt, sp_prompt, ta)            # sequence-parallel prefill, fed the all-reduce run's tokens
    assert tf[0] == ta[0] and sum(a == b for a, b in zip(tf, ta)) >= 5, ("sp vs all-reduce", ta, tf)
    ref = torch.tensor(tb, device=dev)
    dist.broadcast(ref, 0)
    assert ref.tolist() == tb, ("ranks disagree (sp)",)
    del rt

    # a collective that times out (rank 0 calls it alone: nobody raises the flags it waits for), then the group's
    # recovery: epochs re-agreed over NCCL, peer-memory path usable again, and the degraded (library) routing
    late = tp.PeerComm(slot_elems=1 << 16, budget_ms=30.0)
    v = torch.full((2048,), float(rank + 1), device=dev).bfloat16()
    if rank == 0:
        late.all_reduce(v.clone())
        torch.cuda.synchronize()
        try:
            late.check()
            raise AssertionError("expected a collective timeout on rank 0")
        except tp.CollectiveTimeoutError:
            pass
    dist.barrier()
    late.recover(degrade=False)
    want = float(sum(range(1, world + 1)))
    got = late.all_reduce(v.clone())
    torch.cuda.synchronize()
    late.check()
    assert not late.degraded and torch.all(got.float() == want), ("all-reduce after recovery", got[:4])
    late.recover(degrade=True)
    calls0 = late.standalone_calls
    got = late.all_reduce(v.clone())
    torch.cuda.synchronize()
    assert late.degraded and late.standalone_calls == calls0 and torch.all(got.float() == want)
    assert late.sp_rows(1024 * world, 64) == 0
    late.close()

    # expert-parallel combine fused with its collective (one-shot and two-shot) against combine + NCCL
    from deepseek_v4_2080ti_b200.ops import moe
    for t, k, h, rows in [(1, 4, 512, 4), (37, 4, 512, 80), (300, 8, 1024, 900)]:
        torch.manual_seed(21)                     # identical routing on every rank
        owner = torch.randint(0, world, (t, k), device=dev)
        wts = torch.rand(t, k, device=dev)
        resid = torch.randn(t, h, device=dev).bfloat16()
        torch.manual_seed(31 + rank)
        y = torch.randn(rows, h, device=dev).bfloat16()
        base = torch.randn(t, h, device=dev).bfloat16()
        route_row = torch.where(owner == rank, torch.randint(0, rows, (t, k), device=dev), -1).to(torch.int32)
        part = base.float()
        for j in range(k):
            sel = route_row[:, j] >= 0
            part[sel] += wts[sel, j, None] * y[route_row[sel, j].long()].float()
        want = part.bfloat16().float()            # the wire carries bf16 partials
        dist.all_reduce(want)
        want += resid.float()
        for mode in (1, 2):
            got = comm.moe_combine(y, route_row, wts, base, resid, t, k, h, mode)
            torch.cuda.synchronize()
            comm.check()
            err = (got.float() - want).abs().max() / want.abs().max()
            assert err < 2e-2, ("moe_combine", mode, t, err.item())
            ref = got.clone()
            dist.broadcast(ref, 0)
            assert torch.equal(ref, got), ("moe_combine not identical across ranks", mode, t)

    # attention-TP + expert-parallel GGUF model == single-rank model
    from deepseek_v4_2080ti_b200.models import gqa_moe as gm
    gcfg = gm.GqaMoeConfig(n_layers=2, hidden=512, vocab=512, n_heads=2 * world, n_kv_heads=world, n_experts=4 * world,
                           top_k=4, moe_inter=256, context_length=512, attn_type="Q8_0", dense_type="Q4_K",
                           gate_up_type="Q2_K", down_type="IQ2_XXS")
    store = gm.TensorStore(list(gm.synth_tensors(gcfg, seed=9, device=dev, std=0.05)))
    torch.manual_seed(4)
    gprompt = torch.randint(0, gcfg.vocab, (70,), dtype=torch.int32)
    g1 = gm.GqaMoeRuntime(gcfg, gm.GqaMoeGpuWeights(gcfg, store, dev), max_slots=1, max_context=256).generate(gprompt, 8)
    gw = gm.GqaMoeGpuWeights(gcfg, store, dev, rank, world)
    for c, name in ((nccl, "nccl"), (comm, "peer")):
        out = gm.GqaMoeRuntime(gcfg, gw, max_slots=1, max_context=256, comm=c).generate(gprompt, 8, chunk=32)
        torch.cuda.synchronize()
        comm.check()
        assert out[:3] == g1[:3], ("gqa_moe", name, out, g1)
        ref = torch.tensor(out, device=dev)
        dist.broadcast(ref, 0)
        assert ref.tolist() == out, ("gqa_moe ranks disagree", name)
    # MLA + routed-expert family: expert-parallel ranges, and routed tensor parallelism (every rank holds all experts with
    # 1 / world of their width), both against the single-rank model; plus the batched runtime over one page pool
    from deepseek_v4_2080ti_b200.models import mla_moe as mm
    from deepseek_v4_2080ti_b200.models import mla_moe_gpu as mg
    mcfg = mm.MlaMoeConfig(vocab_size=512, hidden_size=256, num_layers=3, first_dense_layers=1, dense_intermediate=256,
                           q_lora_rank=128, kv_lora_rank=128, num_heads=2 * world, qk_nope_dim=64, qk_rope_dim=32,
                           v_head_dim=128, index_heads=4, index_dim=32, index_topk=24, num_experts=2 * world,
                           experts_per_token=2 * world, num_shared_experts=1, expert_intermediate=128 * world,
                           score_func="sigmoid", route_scale=2.5, expert_format="bf16")
    mstate = list(mm.synth_state(mcfg, seed=12, std=0.05))
    mprompt = torch.randint(0, mcfg.vocab_size, (80,), generator=torch.Generator().manual_seed(6), dtype=torch.int32)
    m1, _ = mg.MlaMoeGpuRuntime(mcfg, mg.MlaMoeGpuWeights(mcfg, iter(mstate), dev), max_context=256).generate(mprompt, 6, chunk=32)
    for routed in (False, True):
        mw = mg.MlaMoeGpuWeights(mcfg, iter(mstate), dev, rank=rank, world=world, routed_tp=routed)
        assert mw.routed_tp == routed and (mw.expert_hi - mw.expert_lo) == (mcfg.num_experts if routed else mcfg.num_experts // world)
        out, _ = mg.MlaMoeGpuRuntime(mcfg, mw, max_context=256, comm=comm).generate(mprompt, 6, chunk=32)
        torch.cuda.synchronize()
        comm.check()
        assert out[:3] == m1[:3], ("mla_moe", "routed_tp" if routed else "ep", out, m1)
        ref = torch.tensor(out, device=dev)
        dist.broadcast(ref, 0)
        assert ref.tolist() == out, ("mla_moe ranks disagree", routed)
        if routed:
            brt = mg.MlaMoeBatchRuntime(mcfg, mw, max_slots=2, max_context=256, comm=comm)
            s0, s1 = brt.allocate(), brt.allocate()
            f0, f1 = brt.prefill(s0, mprompt.to(dev), 32), brt.prefill(s1, mprompt[:50].to(dev), 32)
            nxt = brt.decode([s0, s1], torch.cat([f0, f1]).to(torch.int32))
            torch.cuda.synchronize()
            comm.check()
            assert int(f0.item()) == m1[0] and int(nxt[0].item()) == m1[1], ("mla batch", int(f0.item()), nxt.tolist(), m1)
    comm.close()
    dist.barrier()
    if rank == 0:
        print("TP_WORKER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
