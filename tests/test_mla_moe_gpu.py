"""GPU MLA + MoE runtime (absorbed latent attention, indexer top-k, grouped FP4 experts) against the fp32 host runtime."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg(indexer: bool):
    from deepseek_v4_2080ti_b200.models import mla_moe as mm
    return mm.MlaMoeConfig(vocab_size=512, hidden_size=256, num_layers=3, first_dense_layers=1, dense_intermediate=256,
                           q_lora_rank=128, kv_lora_rank=128, num_heads=4, qk_nope_dim=64, qk_rope_dim=32, v_head_dim=128,
                           index_heads=4 if indexer else 0, index_dim=32 if indexer else 0, index_topk=24 if indexer else 0,
                           num_experts=8, experts_per_token=2, num_shared_experts=1, expert_intermediate=128,
                           score_func="sqrtsoftplus", route_scale=1.5)


def test_topk_rows_matches_torch():
    from deepseek_v4_2080ti_b200.ops import mla
    torch.manual_seed(0)
    vals = torch.randn(9, 3000, device="cuda")
    vals[3, 100:140] = 7.0                                  # ties around the threshold
    n = torch.tensor([3000, 2999, 17, 3000, 5, 1024, 2048, 64, 300], dtype=torch.int32, device="cuda")
    k = 64
    idx = mla.topk_rows(vals, n, k)
    for r in range(9):
        got = sorted(i for i in idx[r].tolist() if i >= 0)
        nv = int(n[r])
        if nv <= k:
            assert got == list(range(nv))
            continue
        want_vals = vals[r, :nv].topk(k).values.sort().values
        assert len(got) == k and len(set(got)) == k and max(got) < nv
        assert torch.equal(vals[r, got].sort().values, want_vals)


@pytest.mark.parametrize("indexer", [False, True])
def test_gpu_runtime_follows_host_runtime(indexer):
    from deepseek_v4_2080ti_b200.models import mla_moe as mm
    from deepseek_v4_2080ti_b200.models import mla_moe_gpu as mg
    from deepseek_v4_2080ti_b200.ops import _lib
    cfg = _cfg(indexer)
    state = list(mm.synth_state(cfg, seed=1, std=0.05))
    host = mm.MlaMoeRuntime(cfg, mm.MlaMoeWeights(cfg, iter(state)), max_context=256)
    dev = mg.MlaMoeGpuRuntime(cfg, mg.MlaMoeGpuWeights(cfg, iter(state), "cuda"), max_context=256)
    gen = torch.Generator().manual_seed(2)
    ids = torch.randint(0, cfg.vocab_size, (70,), generator=gen)
    want = torch.cat([host.forward(ids[:50]), host.forward(ids[50:51]), host.forward(ids[51:])])
    got = torch.cat([dev.forward(ids[:50].cuda()), dev.forward(ids[50:51].cuda()), dev.forward(ids[51:].cuda())]).cpu()
    torch.cuda.synchronize()
    _lib.check_status()
    err = (got - want).norm() / want.norm()
    assert err < 6e-2, err
    agree = (got.argmax(-1) == want.argmax(-1)).float().mean().item()
    assert agree > 0.85, agree
