"""Device-side sampling (temperature / top-k / top-p / min-p, penalties) against the fp32 PyTorch restatement, and the
runtime's sampled decoding (seeded reproducibility; top-k 1 equals greedy)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("temperature,top_k,top_p,min_p", [(1.0, 0, 1.0, 0.0), (0.7, 40, 0.9, 0.0), (1.3, 0, 0.5, 0.05),
                                                           (0.2, 5, 1.0, 0.0), (1.0, 1, 1.0, 0.0), (2.0, 1000, 0.95, 0.01)])
def test_sample_matches_reference(temperature, top_k, top_p, min_p):
    from deepseek_v4_2080ti_b200.ops import sampling as smp
    torch.manual_seed(int(temperature * 10) + top_k)
    b, n = 7, 5003
    logits = (torch.randn(b, n, device="cuda") * 3.0).contiguous()
    s = smp.DeviceSampling(temperature, top_k, top_p, min_p)
    for trial in range(3):
        u = torch.rand(b, generator=torch.Generator().manual_seed(trial))
        got = smp.sample(logits, s, u.cuda()).cpu()
        want = smp.sample_ref(logits.cpu(), s, u)
        # a draw that lands within rounding of a CDF step may fall on the neighbouring candidate
        same = (got == want).float().mean().item()
        assert same >= 6 / 7, (got, want)
    if top_k == 1:
        assert torch.equal(got, logits.argmax(-1).cpu().to(torch.int32))


def test_distribution_is_the_tempered_softmax():
    from deepseek_v4_2080ti_b200.ops import sampling as smp
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, -30.0]], device="cuda").repeat(4000, 1).contiguous()
    s = smp.DeviceSampling(temperature=1.5, top_k=4)
    u = torch.rand(4000, generator=torch.Generator().manual_seed(0)).cuda()
    got = smp.sample(logits, s, u).long().cpu()
    freq = torch.bincount(got, minlength=5).float() / 4000
    want = torch.softmax(torch.tensor([2.0, 1.0, 0.0, -1.0]) / 1.5, 0)
    assert freq[4] == 0 and (freq[:4] - want).abs().max() < 0.03, (freq, want)


def test_penalties():
    from deepseek_v4_2080ti_b200.ops import sampling as smp
    logits = torch.tensor([[2.0, -2.0, 1.0, 0.5]], device="cuda")
    counts = torch.tensor([[2, 1, 0, 0]], dtype=torch.int32, device="cuda")
    s = smp.DeviceSampling(1.0, repetition_penalty=2.0, presence_penalty=0.5, frequency_penalty=0.25)
    out = smp.apply_penalties(logits.clone(), counts, s).cpu()
    assert torch.allclose(out, torch.tensor([[2.0 / 2 - 0.5 - 0.5, -2.0 * 2 - 0.5 - 0.25, 1.0, 0.5]]))


def test_runtime_sampled_decoding_is_seeded_and_topk1_is_greedy():
    from types import SimpleNamespace
    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
    from deepseek_v4_2080ti_b200.runtime.loader import RuntimeAdapter
    cfg = qh.QwenHybridConfig.tiny(layers=2)
    w = qh.QwenHybridWeights(cfg, qh.synth_state(cfg, 0, "cuda", std=0.05), "cuda")
    rt = qh.QwenHybridRuntime(cfg, w, max_slots=2, max_context=256)
    ad = RuntimeAdapter(rt, 256)
    prompt = torch.randint(0, cfg.vocab_size, (20,), generator=torch.Generator().manual_seed(1)).tolist()

    def run(sp, n=10):
        slot = ad.allocate()
        out = [ad.prefill_tokens(slot, prompt, 64, sp)]
        for _ in range(n - 1):
            out.append(ad.decode_tokens([slot], [out[-1]], sp)[0])
        ad.free(slot)
        return out

    sp = lambda **k: SimpleNamespace(temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, seed=None, repetition_penalty=1.0,
                                     presence_penalty=0.0, frequency_penalty=0.0, **{}) if not k else \
        SimpleNamespace(**{**dict(temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, seed=None, repetition_penalty=1.0,
                                  presence_penalty=0.0, frequency_penalty=0.0), **k})
    greedy = run(None)
    assert run(sp(top_k=1, seed=3)) == greedy
    a, b, c = run(sp(temperature=1.5, seed=11)), run(sp(temperature=1.5, seed=11)), run(sp(temperature=1.5, seed=12))
    assert a == b and a != c and a != greedy
    pen = run(sp(temperature=0.01, repetition_penalty=1.3, presence_penalty=0.2, seed=1))
    assert all(0 <= t < cfg.vocab_size for t in pen)
