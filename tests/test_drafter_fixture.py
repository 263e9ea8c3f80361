"""The fixture tensor container and the stage-by-stage drafter check: export a fixture from the statement itself, read
it back, and see a changed weight reported at the first stage it touches."""
import json
import struct

import pytest
import torch

from deepseek_v4_2080ti_b200.cli import check_drafter_fixture as chk
from deepseek_v4_2080ti_b200.formats import safetensors_io
from deepseek_v4_2080ti_b200.formats import tensor_file as tf
from deepseek_v4_2080ti_b200.models import qwen_dflash2_ref as df


def test_container_round_trip_and_malformed_files(tmp_path):
    f = tf.TensorFile(11, 42, {"a.b": torch.randn(3, 4), "ids": torch.arange(6).reshape(2, 3), "h": torch.randn(5).to(torch.bfloat16)})
    n = tf.write(tmp_path / "x.qdf2", f)
    raw = (tmp_path / "x.qdf2").read_bytes()
    assert n == len(raw) and raw[:4] == b"QDF2" and struct.unpack_from("<IiiI", raw, 4) == (1, 11, 42, 3)
    g = tf.read(tmp_path / "x.qdf2")
    assert (g.position_offset, g.anchor_token, list(g.tensors)) == (11, 42, ["a.b", "ids", "h"])
    assert torch.equal(g.tensors["a.b"], f.tensors["a.b"]) and g.tensors["ids"].dtype == torch.int32
    assert g.tensors["h"].dtype == torch.float16 and torch.allclose(g.tensors["h"].float(), f.tensors["h"].float(), atol=1e-2)
    (tmp_path / "t.qdf2").write_bytes(raw[:-3])
    with pytest.raises(ValueError, match="payload|truncated"):
        tf.read(tmp_path / "t.qdf2")
    (tmp_path / "m.qdf2").write_bytes(b"XXXX" + raw[4:])
    with pytest.raises(ValueError, match="not a version"):
        tf.read(tmp_path / "m.qdf2")
    (tmp_path / "e.qdf2").write_bytes(raw + b"\0")
    with pytest.raises(ValueError, match="trailing"):
        tf.read(tmp_path / "e.qdf2")
    with pytest.raises(ValueError, match="invalid tensor record"):
        tf.write(tmp_path / "s.qdf2", tf.TensorFile(0, 0, {"scalar": torch.tensor(1.0)}))


def _checkpoints(tmp_path, seed=0):
    cfg = df.QwenDFlash2Config(hidden_size=64, intermediate_size=96, vocab_size=120, num_hidden_layers=2, num_attention_heads=4,
                               num_key_value_heads=2, head_dim=16, block_size=5, conv_group_size=16, conv_kernel_size=2,
                               mask_token_id=119, selector_rank=8, selector_top_k=4, sliding_window=32, target_layer_ids=[0, 2])
    w = df.synth_dflash2_weights(cfg, seed)
    (tmp_path / "drafter").mkdir()
    (tmp_path / "drafter" / "config.json").write_text(json.dumps(cfg.to_json()))
    safetensors_io.write_file(str(tmp_path / "drafter" / "model.safetensors"), w)
    g = torch.Generator().manual_seed(seed + 5)
    tgt = {"model.language_model.embed_tokens.weight": (torch.randn(120, 64, generator=g) * 0.5).to(torch.bfloat16),
           "lm_head.weight": (torch.randn(120, 64, generator=g) * 0.5).to(torch.bfloat16)}
    (tmp_path / "target").mkdir()
    safetensors_io.write_file(str(tmp_path / "target" / "model.safetensors"), tgt)
    taps = torch.randn(9, 128, generator=g)
    tf.write(tmp_path / "capture.qdf2", tf.TensorFile(6, 17, {"target_taps": taps}))
    return cfg, w


def test_export_then_check_passes_and_a_changed_weight_is_located(tmp_path, capsys):
    cfg, w = _checkpoints(tmp_path)
    base = ["--drafter", str(tmp_path / "drafter"), "--target", str(tmp_path / "target")]
    # a capture holds only the taps: nothing to compare, everything to export
    assert chk.main(base + ["--fixture", str(tmp_path / "capture.qdf2"), "--export", str(tmp_path / "full.qdf2")]) == 0
    full = tf.read(tmp_path / "full.qdf2")
    names = list(full.tensors)
    assert names[0] == "target_taps" and names[1:3] == ["context.projected", "context.normalized"]
    for want in ("layer.0.context.k_rope", "noise.tokens", "residual.initial", "layer.1.attention.q_rope", "layer.0.mlp.finish",
                 "layer.1.residual", "final.norm", "logits.local", "topk.global.tokens", "selector.path"):
        assert want in full.tensors, want
    assert full.tensors["noise.tokens"].tolist() == [17, 119, 119, 119, 119] and full.tensors["selector.path"].shape == (4,)
    assert full.tensors["logits.local"].shape == (4, 120) and (full.position_offset, full.anchor_token) == (6, 17)
    capsys.readouterr()
    assert chk.main(base + ["--fixture", str(tmp_path / "full.qdf2"), "--strict-tokens"]) == 0
    out = capsys.readouterr().out
    assert "all within tolerance" in out and f"{len(names) - 1} stages compared" in out
    # the context starts at position 6: rows before it do not exist for the block
    from deepseek_v4_2080ti_b200.cli.check_drafter_fixture import run_stages
    emb, head = chk.find_tensor(str(tmp_path / "target"), "model.language_model.embed_tokens.weight"), chk.find_tensor(str(tmp_path / "target"), "lm_head.weight")
    at0 = run_stages(str(tmp_path / "drafter"), emb, head, full.tensors["target_taps"], 0, 17)
    # rotary attention is relative: moving the whole fixture changes the rotated rows but not what the block computes
    assert (at0["layer.0.attention.q_rope"] - full.tensors["layer.0.attention.q_rope"]).abs().max() > 1e-3
    assert torch.allclose(at0["final.norm"], full.tensors["final.norm"], atol=1e-4)
    # change the MLP of layer 1: everything before it still agrees, the first failure names the stage
    w2 = dict(w)
    w2["layers.1.mlp.up_proj.weight"] = (w["layers.1.mlp.up_proj.weight"].float() * 1.5).to(torch.bfloat16)
    safetensors_io.write_file(str(tmp_path / "drafter" / "model.safetensors"), w2)
    assert chk.main(base + ["--fixture", str(tmp_path / "full.qdf2"), "--json"]) == 1
    rep = json.loads(capsys.readouterr().out)
    bad = [r["stage"] for r in rep["stages"] if r["status"] == "FAIL"]
    assert bad[0] == "layer.1.mlp.up" and "layer.1.mlp.gate" not in bad and "layer.0.residual" not in bad
