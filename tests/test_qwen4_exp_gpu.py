"""GPU runtime of the Qwen4-Exp-style decoder (models/qwen4_exp_gpu.py) against the fp32 host statement of the same
model (models/qwen4_exp_ref.py): chunked prefill that crosses the indexer's dense -> sparse switch, then decode steps."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("budget", [16, 4096])
def test_gpu_runtime_follows_the_host_statement(budget):
    from deepseek_v4_2080ti_b200.models import qwen4_exp_gpu as g4
    from deepseek_v4_2080ti_b200.models import qwen4_exp_ref as q4
    from deepseek_v4_2080ti_b200.ops import _lib
    cfg = q4.Qwen4ExpConfig(hidden_size=128, head_dim=128, num_heads=4, num_kv_heads=2, moe_intermediate=64,
                            shared_intermediate=64, indexer_budget=budget, num_layers=4)
    w = q4.synth_weights(cfg, 2)
    # the device runtime multiplies in bf16: give both models the same bf16-rounded matrices
    w = {k: (v.to(torch.bfloat16).float() if v.dim() == 2 else v) for k, v in w.items()}
    host, dev = q4.Qwen4ExpRef(cfg, w, 128), g4.Qwen4ExpGpu(cfg, w, 128)
    ids = torch.randint(1, cfg.vocab_size, (56,), generator=torch.Generator().manual_seed(4))
    want, got = [], []
    for lo, hi in ((0, 21), (21, 50), (50, 51), (51, 52), (52, 56)):
        want.append(host.forward(ids[lo:hi]))
        got.append(dev.forward(ids[lo:hi]).cpu())
    torch.cuda.synchronize()
    _lib.check_status()
    want, got = torch.cat(want), torch.cat(got)
    assert got.shape == want.shape == (56, cfg.vocab_size) and torch.isfinite(got).all()
    rel = (got - want).norm(dim=-1) / want.norm(dim=-1)
    assert rel.max() < 5e-2, (float(rel.max()), int(rel.argmax()))
    agree = (got.argmax(-1) == want.argmax(-1)).float().mean()
    assert agree >= 0.9, float(agree)
    assert dev.length == host.length == 56


def test_generate_runs_and_matches_host_on_the_first_tokens():
    from deepseek_v4_2080ti_b200.models import qwen4_exp_gpu as g4
    from deepseek_v4_2080ti_b200.models import qwen4_exp_ref as q4
    cfg = q4.Qwen4ExpConfig(hidden_size=128, head_dim=128, moe_intermediate=64, shared_intermediate=64)
    w = {k: (v.to(torch.bfloat16).float() if v.dim() == 2 else v) for k, v in q4.synth_weights(cfg, 7).items()}
    prompt = torch.randint(1, cfg.vocab_size, (30,), generator=torch.Generator().manual_seed(1))
    a = q4.Qwen4ExpRef(cfg, w, 128).generate(prompt, 4, chunk=16)
    b = g4.Qwen4ExpGpu(cfg, w, 128).generate(prompt, 4, chunk=16)
    assert len(b) == 4 and b[0] == a[0]
