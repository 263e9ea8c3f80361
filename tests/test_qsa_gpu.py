"""Sparse-selected grouped-query attention on the GPU (ops/qsa.py) against the fp32 statement, with selections made
by the block-pooled indexer (models/qwen4_exp_components.qsa_select) on the dense and on the sparse path."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("s,past,h,hkv,budget", [(40, 0, 8, 2, 256), (24, 200, 16, 4, 64), (1, 333, 8, 1, 64), (70, 58, 4, 4, 32)])
def test_qsa_attention_matches_fp32(s, past, h, hkv, budget):
    from deepseek_v4_2080ti_b200.models import qwen4_exp_components as C
    from deepseek_v4_2080ti_b200.ops import _lib, qsa
    torch.manual_seed(s + past + h)
    dev = "cuda"
    total = past + s
    k = (torch.randn(total, hkv, 128, device=dev) * 0.5).to(torch.bfloat16)
    v = (torch.randn(total, hkv, 128, device=dev) * 0.5).to(torch.bfloat16)
    q = (torch.randn(s, h, 128, device=dev) * 0.5).to(torch.bfloat16)
    cache = qsa.QsaCache(hkv, total + 5, dev)
    if past:
        cache.append(k[:past], v[:past])
    assert cache.append(k[past:], v[past:]) == past and cache.length == total
    # selections from the indexer's own rule (index queries / keys are random here: any valid selection will do)
    di, hi, ratio = 32, 2, 4
    qi = torch.randn(1, s, hi, di, device=dev)
    raw = torch.randn(1, total, di, device=dev)
    ang = torch.arange(total, device=dev).float()[:, None] * torch.exp(-torch.arange(di // 2, device=dev).float() / 4)[None]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1)[None], torch.cat([ang.sin(), ang.sin()], -1)[None]
    sel = C.qsa_select(qi, raw, torch.ones(di, device=dev), cos, sin, past, budget, ratio)[0].contiguous()
    assert sel.dtype == torch.int32 and sel.shape[0] == s
    pos = torch.arange(past, total, dtype=torch.int32, device=dev)
    # nothing from the future, and no query is left without keys
    assert (sel <= pos[:, None]).all() and (sel >= 0).any(-1).all()
    out = qsa.attention(q, cache, sel, pos)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = qsa.attention_ref(q, k, v, sel)
    assert out.shape == (s, h, 128)
    err = (out.float() - ref).norm() / ref.norm()
    assert err < 1e-2, float(err)
    assert (out.float() - ref).abs().max() < 0.03 * ref.abs().max() + 1e-3
