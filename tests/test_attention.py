"""Paged GQA attention kernels vs an fp32 oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _paged(k, v, bs, extra_blocks=3, seed=0):
    """Scatter contiguous k/v [T, Hkv, 128] into a shuffled paged cache; returns caches + block table row."""
    t, hkv, d = k.shape
    nblk = (t + bs - 1) // bs
    total = nblk + extra_blocks
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(total, generator=g)[:nblk].to(torch.int32)
    kc = torch.zeros(total, hkv, bs, d, dtype=torch.bfloat16, device=k.device)
    vc = torch.zeros_like(kc)
    for i in range(nblk):
        n = min(bs, t - i * bs)
        kc[perm[i], :, :n] = k[i * bs:i * bs + n].transpose(0, 1)
        vc[perm[i], :, :n] = v[i * bs:i * bs + n].transpose(0, 1)
    return kc, vc, perm.to(k.device)


@pytest.mark.parametrize("tq,tk,hq,hkv,bs", [(128, 128, 2, 1, 64), (100, 100, 4, 2, 64), (200, 456, 5, 1, 64),
                                             (384, 384, 8, 8, 16), (50, 1000, 6, 2, 128), (1, 300, 5, 1, 32)])
@pytest.mark.parametrize("use_gate", [False, True])
def test_prefill(tq, tk, hq, hkv, bs, use_gate):
    from deepseek_v4_2080ti_b200.ops import _lib, attention
    torch.manual_seed(tq + tk)
    q = torch.randn(tq, hq, 128, device="cuda").bfloat16()
    k = torch.randn(tk, hkv, 128, device="cuda").bfloat16()
    v = torch.randn(tk, hkv, 128, device="cuda").bfloat16()
    gate = torch.randn(tq, hq, 128, device="cuda").bfloat16() if use_gate else None
    kc, vc, row = _paged(k, v, bs)
    bt = row[None].contiguous()
    i32 = lambda x: torch.tensor([x], dtype=torch.int32, device="cuda")
    out = attention.prefill(q, kc, vc, bt, i32(0), i32(tq), i32(tk), tq, gate=gate)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = attention.attention_ref(q, k, v, tk - tq, gate)
    err = (out.float() - ref).abs().max().item()
    assert err < 3e-2, err


def test_prefill_two_sequences():
    from deepseek_v4_2080ti_b200.ops import _lib, attention
    torch.manual_seed(9)
    lens = [(70, 200), (130, 130)]
    hq, hkv, bs = 4, 2, 64
    qs, refs, rows = [], [], []
    caches = []
    for i, (tq, tk) in enumerate(lens):
        q = torch.randn(tq, hq, 128, device="cuda").bfloat16()
        k = torch.randn(tk, hkv, 128, device="cuda").bfloat16()
        v = torch.randn(tk, hkv, 128, device="cuda").bfloat16()
        qs.append(q)
        refs.append(attention.attention_ref(q, k, v, tk - tq))
        caches.append(_paged(k, v, bs, extra_blocks=0, seed=i))
    # merge the two caches into one pool
    kc = torch.cat([c[0] for c in caches])
    vc = torch.cat([c[1] for c in caches])
    off = caches[0][0].shape[0]
    mb = max(c[2].numel() for c in caches)
    bt = torch.zeros(2, mb, dtype=torch.int32, device="cuda")
    bt[0, :caches[0][2].numel()] = caches[0][2]
    bt[1, :caches[1][2].numel()] = caches[1][2] + off
    t = lambda xs: torch.tensor(xs, dtype=torch.int32, device="cuda")
    out = attention.prefill(torch.cat(qs), kc, vc, bt, t([0, 70]), t([70, 130]), t([200, 130]), 130)
    torch.cuda.synchronize()
    _lib.check_status()
    assert (out[:70].float() - refs[0]).abs().max().item() < 3e-2
    assert (out[70:].float() - refs[1]).abs().max().item() < 3e-2


@pytest.mark.parametrize("b,tk,hq,hkv,bs,splits", [(1, 77, 5, 1, 64, 1), (3, 1000, 8, 2, 16, 4), (2, 4096, 6, 1, 64, None),
                                                    (4, 130, 4, 4, 64, 2)])
def test_decode(b, tk, hq, hkv, bs, splits):
    from deepseek_v4_2080ti_b200.ops import attention
    torch.manual_seed(b * tk)
    outs, refs = [], []
    pools, rows = [], []
    q = torch.randn(b, hq, 128, device="cuda").bfloat16()
    gate = torch.randn(b, hq, 128, device="cuda").bfloat16()
    lens = [max(1, tk - 13 * i) for i in range(b)]
    for i in range(b):
        k = torch.randn(lens[i], hkv, 128, device="cuda").bfloat16()
        v = torch.randn(lens[i], hkv, 128, device="cuda").bfloat16()
        refs.append(attention.attention_ref(q[i:i + 1], k, v, lens[i] - 1, gate[i:i + 1]))
        pools.append(_paged(k, v, bs, extra_blocks=1, seed=i))
    kc = torch.cat([p[0] for p in pools])
    vc = torch.cat([p[1] for p in pools])
    mb = max(p[2].numel() for p in pools)
    bt = torch.zeros(b, mb, dtype=torch.int32, device="cuda")
    off = 0
    for i, p in enumerate(pools):
        bt[i, :p[2].numel()] = p[2] + off
        off += p[0].shape[0]
    kv_len = torch.tensor(lens, dtype=torch.int32, device="cuda")
    out = attention.decode(q, kc, vc, bt, kv_len, gate=gate, splits=splits, max_kv_len=tk)
    err = (out.float() - torch.cat(refs)).abs().max().item()
    assert err < 2e-2, err


def test_qk_norm_rope_append():
    from deepseek_v4_2080ti_b200.ops import attention, basic
    torch.manual_seed(11)
    t, hq, hkv, bs, rot = 37, 4, 2, 16, 64
    width = hq * 256 + 2 * hkv * 128
    src = torch.randn(t, width, device="cuda").bfloat16()
    qg = (torch.randn(128, device="cuda") * 0.1).bfloat16()
    kg = (torch.randn(128, device="cuda") * 0.1).bfloat16()
    inv = attention.rope_inv_freq(rot, 1e7, "cuda")
    pos = torch.arange(1000, 1000 + t, dtype=torch.int32, device="cuda")
    nblk = (t + bs - 1) // bs
    blocks = torch.randperm(nblk + 2)[:nblk].to(torch.int32).cuda()
    slots = (blocks[torch.arange(t, device="cuda") // bs] * bs + torch.arange(t, device="cuda") % bs).to(torch.int32)
    kc = torch.zeros(nblk + 2, hkv, bs, 128, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    q, gate = attention.qk_norm_rope_append(src, 0, 256, True, src, hq * 256, src, hq * 256 + hkv * 128, qg, kg, True,
                                            1e-6, inv, rot, pos, slots, kc, vc, hq, hkv)
    qsrc = src[:, :hq * 256].view(t, hq, 256)
    want_q = attention.rope_ref(basic.rmsnorm_ref(qsrc[..., :128], qg, 1e-6, True), pos, inv, rot)
    assert (q.float() - want_q).abs().max().item() < 3e-2
    assert torch.equal(gate, qsrc[..., 128:].contiguous())
    ksrc = src[:, hq * 256:hq * 256 + hkv * 128].view(t, hkv, 128)
    vsrc = src[:, hq * 256 + hkv * 128:].view(t, hkv, 128)
    want_k = attention.rope_ref(basic.rmsnorm_ref(ksrc, kg, 1e-6, True), pos, inv, rot)
    got_k = kc[(slots // bs).long(), :, (slots % bs).long()]
    got_v = vc[(slots // bs).long(), :, (slots % bs).long()]
    assert (got_k.float() - want_k).abs().max().item() < 3e-2
    assert torch.equal(got_v, vsrc)


@pytest.mark.parametrize("window,sinks", [(64, 0), (100, 4), (300, 130), (16, 16)])
def test_sliding_window_with_sinks_prefill_and_decode(window, sinks):
    """A query at position p sees keys (p - window, p] and the first `sinks` keys; prefill (with tile skipping) and
    split-KV decode against fp32 PyTorch with the same mask, on a scrambled page table."""
    from deepseek_v4_2080ti_b200.ops import _lib, attention
    torch.manual_seed(window + sinks)
    hq, hkv, bs, ctx, tq = 4, 2, 64, 700, 450
    nblk = (ctx + bs - 1) // bs
    perm = torch.randperm(nblk) + 1
    bt = perm.to(torch.int32).cuda().view(1, nblk).contiguous()
    kc = torch.zeros(nblk + 1, hkv, bs, 128, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    k = (torch.randn(ctx, hkv, 128, device="cuda") * 0.5).bfloat16()
    v = (torch.randn(ctx, hkv, 128, device="cuda") * 0.5).bfloat16()
    pos = torch.arange(ctx)
    blk, off = perm[pos // bs].cuda(), (pos % bs).cuda()
    kc[blk, :, off] = k
    vc[blk, :, off] = v
    q = (torch.randn(tq, hq, 128, device="cuda") * 0.5).bfloat16()
    i32 = lambda x: torch.tensor([x], dtype=torch.int32, device="cuda")
    out = attention.prefill(q, kc, vc, bt, i32(0), i32(tq), i32(ctx), tq, window=window, sinks=sinks)
    qpos = torch.arange(ctx - tq, ctx, device="cuda")
    kpos = torch.arange(ctx, device="cuda")
    vis = (kpos[None] <= qpos[:, None]) & ((kpos[None] > qpos[:, None] - window) | (kpos[None] < sinks))
    kk, vv = k.float().repeat_interleave(hq // hkv, 1), v.float().repeat_interleave(hq // hkv, 1)
    sc = torch.einsum("qhd,khd->hqk", q.float(), kk) / 128 ** 0.5
    want = torch.einsum("hqk,khd->qhd", sc.masked_fill(~vis[None], float("-inf")).softmax(-1), vv)
    torch.cuda.synchronize()
    _lib.check_status()
    assert (out.float() - want).abs().max() < 2e-2
    for splits in (1, 3):
        qd = q[-1:].contiguous()
        od = attention.decode(qd, kc, vc, bt, i32(ctx), splits=splits, window=window, sinks=sinks)
        assert (od.float() - want[-1:]).abs().max() < 2e-2, splits


@pytest.mark.parametrize("fmt,tol_k,tol_v", [("fp8", 0.04, 0.04), ("int8_per_token_head", 0.015, 0.015),
                                              ("turboquant_k8v4", 0.04, 0.16)])
def test_kv8_cache_roundtrip_and_decode(fmt, tol_k, tol_v):
    """Quantising append into the quantised cache, its dequantisation back to staging, and decode attention reading
    the quantised rows directly (against the fp32 oracle on the dequantised rows)."""
    from deepseek_v4_2080ti_b200.ops import _lib, attention
    torch.manual_seed(5)
    hkv, hq, bs, t = 2, 6, 64, 333
    nblk = (t + bs - 1) // bs
    k = (torch.randn(t, hkv, 128, device="cuda") * torch.rand(t, hkv, 1, device="cuda") * 3).bfloat16()
    v = (torch.randn(t, hkv, 128, device="cuda") + 0.3).bfloat16()
    stage_k = torch.zeros(nblk, hkv, bs, 128, dtype=torch.bfloat16, device="cuda")
    stage_v = torch.zeros_like(stage_k)
    pos = torch.arange(t, device="cuda")
    stage_k[pos // bs, :, pos % bs] = k
    stage_v[pos // bs, :, pos % bs] = v
    cache = attention.Kv8Cache(fmt, 1, nblk + 4, hkv, bs, "cuda")
    k8, v8, ks, vs, vm = cache.layer(0)
    assert v8.shape[-1] == (64 if fmt == "turboquant_k8v4" else 128)
    perm = torch.randperm(nblk + 3, device="cuda")[:nblk].to(torch.int32) + 1
    dst = (perm[(pos // bs).long()] * bs + pos % bs).to(torch.int32)
    src = pos.to(torch.int32)
    src[7], dst[7] = -1, -1                               # skipped row stays zero
    attention.kv8_quantize(cache.fmt, stage_k, stage_v, src, dst, k8, v8, ks, vs, vm)
    back_k, back_v = torch.zeros_like(stage_k), torch.zeros_like(stage_v)
    attention.kv8_dequantize(cache.fmt, k8, v8, ks, vs, perm, t, back_k, back_v, vm)
    torch.cuda.synchronize()
    _lib.check_status()
    kd = back_k[pos // bs, :, pos % bs].float()
    vd = back_v[pos // bs, :, pos % bs].float()
    assert kd[7].abs().max().item() == 0
    keep = torch.ones(t, dtype=torch.bool, device="cuda")
    keep[7] = False
    for got, want, tol in ((kd, k.float(), tol_k), (vd, v.float(), tol_v)):
        rel = (got[keep] - want[keep]).norm(dim=-1) / want[keep].norm(dim=-1)
        assert rel.max().item() < tol, rel.max().item()
    q = torch.randn(1, hq, 128, device="cuda").bfloat16()
    gate = torch.randn(1, hq, 128, device="cuda").bfloat16()
    kv_len = torch.tensor([t], dtype=torch.int32, device="cuda")
    # the oracle sees the cache's exact values (scale * code, before the staging copy's bf16 rounding)
    pl = perm.long()

    def codes(c8):
        if fmt == "int8_per_token_head":
            return c8[pl].view(torch.int8).float()
        return c8[pl].view(torch.float8_e4m3fn).float()

    fk = codes(k8) * ks[pl][..., None]
    if fmt == "turboquant_k8v4":
        nib = torch.stack([v8[pl] & 15, v8[pl] >> 4], -1).flatten(-2).float()          # even dim in the low nibble
        fv = nib * vs[pl][..., None] + vm[pl][..., None]
    else:
        fv = codes(v8) * vs[pl][..., None]
    fk = fk.permute(0, 2, 1, 3).reshape(-1, hkv, 128)[:t]
    fv = fv.permute(0, 2, 1, 3).reshape(-1, hkv, 128)[:t]
    ref = attention.attention_ref(q, fk, fv, t - 1, gate)
    bt = perm[None].contiguous()
    for splits in (1, 3):
        out = attention.decode_kv8(cache.fmt, q, k8, v8, ks, vs, bt, kv_len, gate=gate, splits=splits, max_kv_len=t, v_min=vm)
        assert (out.float() - ref).abs().max().item() < 2e-2
    win = attention.decode_kv8(cache.fmt, q, k8, v8, ks, vs, bt, kv_len, splits=2, max_kv_len=t, window=64, sinks=4, v_min=vm)
    vis = torch.cat([torch.arange(4, device="cuda"), torch.arange(t - 64, t, device="cuda")])
    ref_w = attention.attention_ref(q, fk[vis], fv[vis], vis.numel() - 1)
    assert (win.float() - ref_w).abs().max().item() < 2e-2
