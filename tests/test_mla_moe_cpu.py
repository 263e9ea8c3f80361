"""Tiny DeepSeek-style decoder on the CPU: the cached, absorbed-MLA runtime with FP4 routed experts executed by
the host kernels must reproduce the fp32 PyTorch oracle token for token (greedy) and logit for logit."""
import torch

from deepseek_v4_2080ti_b200.formats import fp4 as fp4fmt
from deepseek_v4_2080ti_b200.models import mla_moe as mm
from deepseek_v4_2080ti_b200.models.reference_cpu.mla_moe_ref import MlaMoeRef


def test_fp4_roundtrip_and_layout():
    torch.manual_seed(0)
    w = torch.randn(48, 128) * 0.02
    q, s = fp4fmt.quantize(w)
    assert q.shape == (48, 64) and s.shape == (48, 4) and q.dtype == torch.uint8
    d = fp4fmt.dequantize(q, s)
    assert (d - w).abs().max() <= 0.26 * w.abs().max()      # half a level step at the top of the range
    # low nibble holds the even element
    codes = fp4fmt.unpack_codes(q)
    assert torch.equal(codes[:, 0], q[:, 0] & 0xF) and torch.equal(codes[:, 1], q[:, 0] >> 4)
    assert float(fp4fmt.level_table()[5]) == 3.0 and float(fp4fmt.level_table()[15]) == -6.0


def test_cpu_fp4_moe_matches_dequantised_loop():
    torch.manual_seed(1)
    t, h, inter, e, k = 7, 256, 128, 8, 2
    x = torch.randn(t, h)
    ws = [[fp4fmt.quantize(torch.randn(*shape) * 0.05) for shape in ((inter, h), (inter, h), (h, inter))] for _ in range(e)]
    w13 = torch.stack([torch.cat([w[0][0], w[1][0]]) for w in ws])
    s13 = torch.stack([torch.cat([w[0][1], w[1][1]]) for w in ws])
    w2 = torch.stack([w[2][0] for w in ws])
    s2 = torch.stack([w[2][1] for w in ws])
    idx = torch.stack([torch.randperm(e)[:k] for _ in range(t)]).to(torch.int32)
    idx[3, 1] = -1                                          # a route owned by another rank
    wts = torch.rand(t, k)
    got = mm.cpu_moe_fp4(x, idx, wts, w13, s13, w2, s2, inter, swiglu_limit=4.0, threads=3)
    want = torch.zeros(t, h)
    for ti in range(t):
        for ki in range(k):
            ei = int(idx[ti, ki])
            if ei < 0:
                continue
            w1, w3, wd = (fp4fmt.dequantize(*ws[ei][j]) for j in range(3))
            want[ti] += wts[ti, ki] * mm.swiglu(x[ti:ti + 1], w1, w3, wd, 4.0)[0]
    assert (got - want).abs().max() <= 1e-4 * want.abs().max().clamp_min(1e-6)
    # thread count does not change a single bit
    again = mm.cpu_moe_fp4(x, idx, wts, w13, s13, w2, s2, inter, swiglu_limit=4.0, threads=1)
    assert torch.equal(got, again)


def test_tiny_model_token_and_logit_parity():
    cfg = mm.MlaMoeConfig.tiny_cpu()
    state = list(mm.synth_state(cfg, seed=0))
    assert any(k.endswith("experts.0.w1.scale") for k, _ in state)
    rt = mm.MlaMoeRuntime(cfg, mm.MlaMoeWeights(cfg, iter(state)), max_context=128)
    ref = MlaMoeRef(cfg, state)
    gen = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab_size, (64,), generator=gen)
    toks, logits = rt.generate(prompt, 16)
    want_toks, want_logits = ref.generate(prompt, 16)
    assert toks == want_toks
    err = (logits - want_logits).abs().max() / want_logits.abs().max()
    assert err < 1e-4, err


def test_indexer_selection_matches_oracle():
    """With an indexer and a context longer than top-k, cached decode picks the same keys as the oracle."""
    cfg = mm.MlaMoeConfig.tiny_cpu()
    cfg.index_heads, cfg.index_dim, cfg.index_topk = 4, 32, 16
    state = list(mm.synth_state(cfg, seed=2))
    rt = mm.MlaMoeRuntime(cfg, mm.MlaMoeWeights(cfg, iter(state)), max_context=128)
    ref = MlaMoeRef(cfg, state)
    gen = torch.Generator().manual_seed(3)
    ids = torch.randint(0, cfg.vocab_size, (40,), generator=gen)
    got = torch.cat([rt.forward(ids[:30]), rt.forward(ids[30:31]), rt.forward(ids[31:])])
    want = ref.forward(ids)
    # prefill rows with fewer visible keys than top-k see everything in both implementations
    assert (got - want).abs().max() / want.abs().max() < 1e-4


def test_expert_parallel_ranks_sum_to_full_model():
    """Each expert-parallel rank holds a contiguous expert range and skips routes it does not own; the rank
    outputs for the same layer input add up to the single-rank routed output."""
    cfg = mm.MlaMoeConfig.tiny_cpu()
    state = list(mm.synth_state(cfg, seed=4))
    full = mm.MlaMoeRuntime(cfg, mm.MlaMoeWeights(cfg, iter(state)), max_context=64)
    ranks = [mm.MlaMoeRuntime(cfg, mm.MlaMoeWeights(cfg, iter(state), ep_rank=r, ep_world=2), max_context=64)
             for r in range(2)]
    assert (ranks[1].w.expert_lo, ranks[1].w.expert_hi) == (4, 8)
    ids = torch.randint(0, cfg.vocab_size, (20,), generator=torch.Generator().manual_seed(5))
    x = mm.rms_norm(full.w.embed[ids.long()].float(), full.w.layers[0].ffn_norm, cfg.rms_norm_eps)
    for i, lw in enumerate(full.w.layers):
        want = full._ffn(lw, x)
        shared = mm.swiglu(x, *[m.float() for m in lw.shared])
        parts = []
        for r in ranks:
            rl = r.w.layers[i]
            rl.shared = None
            parts.append(r._ffn(rl, x))
        assert (parts[0] + parts[1] + shared - want).abs().max() <= 1e-5 * want.abs().max()
