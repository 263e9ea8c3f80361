"""Safetensors writer/reader round trip, shard index, and agreement with the C++ reader."""
import json
import os

import pytest
import torch

from deepseek_v4_2080ti_b200.formats import fp8 as fp8fmt
from deepseek_v4_2080ti_b200.formats import safetensors_io as st


def test_roundtrip_dtypes_and_sharding(tmp_path):
    torch.manual_seed(0)
    w = torch.randn(256, 384) * 0.02
    q, s = fp8fmt.quantize_block128(w)
    state = {"a.weight": q, "a.weight_scale_inv": s, "b": torch.randn(7, 3).bfloat16(), "c": torch.arange(5, dtype=torch.int32),
             "d": torch.randn(300, 300)}
    files = st.write_checkpoint(str(tmp_path), state.items(), shard_bytes=200_000, config_json="{}")
    assert len(files) >= 2 and os.path.exists(tmp_path / "config.json")
    idx = json.load(open(tmp_path / "model.safetensors.index.json"))
    assert set(idx["weight_map"]) == set(state)
    back = dict(st.read_checkpoint(str(tmp_path)))
    for k, v in state.items():
        assert back[k].dtype == v.dtype and back[k].shape == v.shape
        assert torch.equal(back[k].view(torch.uint8), v.contiguous().view(torch.uint8))
    assert (fp8fmt.dequantize_block128(back["a.weight"], back["a.weight_scale_inv"]) - w).abs().max() < 0.02 * 0.07 * 4


def test_cpp_reader_sees_the_same_bytes(tmp_path):
    cpp = pytest.importorskip("deepseek_v4_2080ti_b200.pocketllm_cpp")
    t = torch.randn(64, 32).bfloat16()
    st.write_checkpoint(str(tmp_path), [("x.weight", t)])
    ws = cpp.WeightSource.open(str(tmp_path))
    v = ws.get("x.weight")
    assert v["dtype"] == "BF16" and v["shape"] == [64, 32]
    assert bytes(v["data"]) == t.view(torch.uint8).numpy().tobytes()


def test_qwen_synthetic_checkpoint_on_disk_matches_generator(tmp_path):
    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
    cfg = qh.QwenHybridConfig.tiny(layers=2)
    st.write_checkpoint(str(tmp_path), qh.synth_state(cfg, 3, "cpu"), config_json=cfg.to_json())
    cfg2 = qh.QwenHybridConfig.from_json(tmp_path / "config.json")
    assert cfg2.layer_types == cfg.layer_types and cfg2.rope_theta == cfg.rope_theta and cfg2.hidden_size == 256
    disk = dict(st.read_checkpoint(str(tmp_path)))
    for name, t in qh.synth_state(cfg, 3, "cpu"):
        assert torch.equal(disk[name].view(torch.uint8), t.view(torch.uint8)), name
    names = {n for n, _, _ in qh.tensor_specs(cfg)}
    assert "model.language_model.layers.0.linear_attn.in_proj_qkv.weight" in names
    assert "model.language_model.layers.1.self_attn.q_proj.weight" in names
