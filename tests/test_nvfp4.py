"""NVFP4 weights (E2M1, E4M3 scale per 16, fp32 global scale): format round trips on CPU; on a GPU, a hybrid checkpoint
whose feed-forward matrices are NVFP4 (attention stays FP8) against the fp32 oracle."""
import pytest
import torch


def _to_nvfp4_state(state, layers):
    """Replace the MLP matrices of ``layers`` by NVFP4 tensors quantised from the dequantised FP8 weights."""
    from deepseek_v4_2080ti_b200.formats import fp8 as fp8fmt
    from deepseek_v4_2080ti_b200.formats import nvfp4
    raw = dict(state)
    out = []
    for k, v in state:
        hit = any(f"layers.{i}.mlp." in k for i in layers)
        if hit and k.endswith(".weight_scale_inv"):
            continue
        if hit and k.endswith(".weight"):
            base = k[:-len(".weight")]
            w = fp8fmt.dequantize_block128(v.cpu(), raw[k + "_scale_inv"].cpu())
            p, s, g = nvfp4.quantize(w)
            out += [(base + ".weight_packed", p), (base + ".weight_scale", s), (base + ".weight_global_scale", g),
                    (base + ".input_global_scale", torch.ones(1))]
            continue
        out.append((k, v))
    return out


def test_quantise_dequantise_and_block64_records():
    from deepseek_v4_2080ti_b200.formats import nvfp4
    torch.manual_seed(0)
    w = torch.randn(48, 256) * 0.05
    w[3] *= 20                                              # one row with a much larger range
    p, s, g = nvfp4.quantize(w)
    assert p.shape == (48, 128) and p.dtype == torch.uint8 and s.shape == (48, 16) and s.dtype == torch.float8_e4m3fn
    d = nvfp4.dequantize(p, s, g)
    assert ((d - w).norm() / w.norm()).item() < 0.13
    p2, s2, g2 = nvfp4.quantize(d)                          # representable values survive a second pass
    assert torch.equal(nvfp4.dequantize(p2, s2, g2), d)
    # low nibble is the earlier weight
    one = torch.zeros(1, 16)
    one[0, 0], one[0, 1] = 6.0, -3.0
    pk, sk, gk = nvfp4.quantize(one)
    assert pk[0, 0].item() == (0x7 | (0xD << 4)) and nvfp4.dequantize(pk, sk, gk)[0, :2].tolist() == [6.0, -3.0]
    rec = nvfp4.to_block64(p, s)
    assert rec.shape == (48, 4, 36)
    pp, ss = nvfp4.from_block64(rec)
    assert torch.equal(pp, p) and torch.equal(ss.view(torch.uint8), s.view(torch.uint8))


def test_oracle_reads_a_mixed_nvfp4_checkpoint():
    from deepseek_v4_2080ti_b200.formats import nvfp4
    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
    from deepseek_v4_2080ti_b200.models.reference_cpu.qwen_hybrid_ref import QwenHybridRef
    cfg = qh.QwenHybridConfig.tiny(layers=2)
    state = list(qh.synth_state(cfg, 0, "cpu", std=0.05))
    mixed = _to_nvfp4_state(state, layers=(0,))
    names = {k for k, _ in mixed}
    assert "model.language_model.layers.0.mlp.up_proj.weight_packed" in names
    assert "model.language_model.layers.1.mlp.up_proj.weight" in names
    ref = QwenHybridRef(cfg, mixed)
    raw = dict(mixed)
    base = "model.language_model.layers.0.mlp.down_proj"
    want = nvfp4.dequantize(raw[base + ".weight_packed"], raw[base + ".weight_scale"], raw[base + ".weight_global_scale"])
    assert torch.equal(ref.p[base + ".weight"], want)
    ids = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(1), dtype=torch.int32)
    assert torch.isfinite(ref.forward(ids)).all()


def test_weight_map_audit_accepts_nvfp4_feed_forward_matrices():
    import os
    import tempfile
    from deepseek_v4_2080ti_b200 import pocketllm_cpp as core
    from deepseek_v4_2080ti_b200.formats import safetensors_io
    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
    cfg = qh.QwenHybridConfig.tiny(layers=2)
    mixed = _to_nvfp4_state(list(qh.synth_state(cfg, 0, "cpu", std=0.05)), layers=(0,))
    with tempfile.TemporaryDirectory() as d:
        safetensors_io.write_checkpoint(d, iter(mixed), config_json=cfg.to_json())
        rep = core.qwen_audit(d, 1)
        assert rep["ok"] and rep["ok_strict"], rep
    with tempfile.TemporaryDirectory() as d:
        bad = [(k, v) for k, v in mixed if not k.endswith("layers.0.mlp.up_proj.weight_global_scale")]
        safetensors_io.write_checkpoint(d, iter(bad), config_json=cfg.to_json())
        rep = core.qwen_audit(d, 1)
        assert rep["missing"] == ["model.language_model.layers.0.mlp.up_proj.weight_global_scale"]


@pytest.mark.gpu
def test_runtime_with_nvfp4_feed_forward_matches_the_oracle():
    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
    from deepseek_v4_2080ti_b200.models.reference_cpu.qwen_hybrid_ref import QwenHybridRef
    from deepseek_v4_2080ti_b200.ops import _lib, gemm
    cfg = qh.QwenHybridConfig.tiny(layers=4)
    state = list(qh.synth_state(cfg, 0, "cuda", std=0.05))
    mixed = _to_nvfp4_state(state, layers=(0, 1, 2))        # the last layer keeps its FP8 feed-forward
    w = qh.QwenHybridWeights(cfg, iter(mixed), "cuda")
    assert w.layers[0].gate_up.wfmt == gemm.WF_BF16 and w.layers[3].gate_up.wfmt == gemm.WF_FP8_B128
    rt = qh.QwenHybridRuntime(cfg, w, max_slots=1, max_context=256)
    assert not rt.fused_decode
    ref = QwenHybridRef(cfg, [(k, v.cpu()) for k, v in mixed])
    ids = torch.randint(0, cfg.vocab_size, (90,), generator=torch.Generator().manual_seed(2), dtype=torch.int32).cuda()
    want = ref.forward(ids.cpu())
    slot = rt.allocate()
    nxt = rt.prefill(slot, ids, chunk=64)
    torch.cuda.synchronize()
    _lib.check_status()
    got = rt.last_logits.float()[0]
    assert torch.nn.functional.cosine_similarity(got, want[-1].to(got.device), dim=0).item() > 0.995
    tok = rt.decode([slot], nxt.to(torch.int32))
    assert 0 <= int(tok.item()) < cfg.vocab_size
