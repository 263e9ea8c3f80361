"""Host-side tools: importance-matrix capture / merge, page-cache prewarm, family registry and the GGUF CLIs."""
import json
import os
import tempfile

import torch

from deepseek_v4_2080ti_b200.formats import gguf as G
from deepseek_v4_2080ti_b200.formats.gguf import imatrix, prewarm
from deepseek_v4_2080ti_b200.models import gqa_moe as gm
from deepseek_v4_2080ti_b200.models import registry


def test_imatrix_collect_merge_round_trip():
    torch.manual_seed(0)
    c1 = imatrix.RoutedIMatrixCollector(n_experts=4, chunk_size=8)
    c2 = imatrix.RoutedIMatrixCollector(n_experts=4, chunk_size=8, layers={0})
    x = torch.randn(10, 16)
    c1.observe(0, 2, "ffn_gate_exps", x)
    c1.observe(1, 9, "ffn_gate_exps", x)                   # out-of-range expert: ignored
    # sorted rows: expert 1 gets rows 0:3, expert 3 rows 3:7; the last 3 rows are padding
    offsets = torch.tensor([0, 0, 3, 3, 7])
    c1.observe_sorted(0, "ffn_down_exps", x, offsets)
    c2.observe_sorted(0, "ffn_down_exps", x, torch.tensor([0, 2, 2]), expert_lo=2)   # a rank holding experts 2..3
    c2.observe(5, 0, "ffn_gate_exps", x)                   # layer filtered out
    with tempfile.TemporaryDirectory() as d:
        p1, p2, pm = (os.path.join(d, n) for n in ("a.gguf", "b.gguf", "m.gguf"))
        r1 = c1.save(p1)
        c2.save(p2)
        assert r1["entries"] == 2 and r1["chunk_count"] == 2            # max count 10 rows / chunk 8
        e1, meta = imatrix.read_imatrix(p1)
        assert meta["general.type"] == "imatrix" and meta["imatrix.chunk_size"] == 8
        s2, cnt = e1["blk.0.ffn_gate_exps.weight"]
        assert torch.allclose(s2[2], (x * x).sum(0)) and cnt.tolist() == [0, 0, 10, 0]
        s2, cnt = e1["blk.0.ffn_down_exps.weight"]
        assert cnt.tolist() == [0, 3, 0, 4] and torch.allclose(s2[3], (x[3:7] ** 2).sum(0))
        imatrix.merge_imatrix_files([p1, p2], pm)
        em, _ = imatrix.read_imatrix(pm)
        s2, cnt = em["blk.0.ffn_down_exps.weight"]
        assert cnt.tolist() == [0, 3, 2, 4] and torch.allclose(s2[2], (x[:2] ** 2).sum(0), atol=1e-5)
        from deepseek_v4_2080ti_b200.cli import merge_imatrix as cli
        assert cli.main([p1, p2, "-o", os.path.join(d, "m2.gguf")]) == 0
    assert imatrix.rank_output_path("x.gguf", 3, 8) == "x.rank3.gguf" and imatrix.rank_output_path("x{rank}.gguf", 3, 8) == "x3.gguf"
    assert imatrix.rank_output_path("x.gguf", 0, 1) == "x.gguf"


def _tiny_gguf(d):
    cfg = gm.GqaMoeConfig.tiny(layers=1, experts=4)
    cfg.gate_up_type, cfg.down_type = "Q2_K", "Q2_K"
    path = os.path.join(d, "tiny.gguf")
    gm.write_synthetic_gguf(path, cfg, seed=1)
    return cfg, path


def test_prewarm_reads_files_and_tensor_ranges():
    with tempfile.TemporaryDirectory() as d:
        cfg, path = _tiny_gguf(d)
        r = prewarm.prewarm_paths([path], threads=2, chunk_bytes=4096)
        assert r["files"] == 1 and r["bytes"] == os.path.getsize(path)
        b = G.read_bundle(path)
        names = {"blk.0.ffn_gate_exps.weight", "output.weight"}
        r = prewarm.prewarm_bundle(b, names)
        assert r["bytes"] == sum(b.tensors[n].nbytes for n in names)
        assert prewarm.prewarm_paths([path], max_bytes=10000, chunk_bytes=4096)["bytes"] <= 10000 + 4096


def test_registry_validates_reports_capability_and_plans_placement(capsys):
    with tempfile.TemporaryDirectory() as d:
        cfg, path = _tiny_gguf(d)
        b = G.read_bundle(path)
        spec = registry.detect(b)
        assert spec.architecture == "minimax-m2" and "minimax-m2" in registry.architectures()
        rep = spec.validate(b)
        assert rep.ok and not rep.missing and not rep.unexpected and rep.routed_bytes > 0
        assert set(rep.by_type) == {"Q4_K", "Q5_K", "Q2_K", "F32"}
        plan = spec.placement(rep, registry.HardwareProfile(8, 180.0))
        assert plan[0].name == "all_device_resident" and plan[0].status == "candidate"
        small = spec.placement(rep, registry.HardwareProfile(1, 0.0001))
        assert small[0].status == "rejected" and small[1].name == "layer_pipeline"
        assert registry.capability_status(G.GGMLType.IQ1_M)[0] == "supported"
        assert registry.capability_status(G.GGMLType.Q6_K)[0] == "supported"
        from deepseek_v4_2080ti_b200.cli import inspect_gguf, make_routed_source_gguf
        assert inspect_gguf.main([path, "--validate", "--placement", "--json"]) == 0
        out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
        assert out["architecture"] == "minimax-m2" and out["validation"]["ok"] and out["capability"]["Q5_K"] == "supported"
        routed = os.path.join(d, "routed.gguf")
        assert make_routed_source_gguf.main([path, "-o", routed, "--experts", "1:3"]) == 0
        rb = G.read_bundle(routed)
        assert set(rb.tensors) == {"blk.0.ffn_gate_exps.weight", "blk.0.ffn_up_exps.weight", "blk.0.ffn_down_exps.weight"}
        assert rb.tensors["blk.0.ffn_gate_exps.weight"].shape[0] == 2
        assert torch.equal(rb.raw("blk.0.ffn_up_exps.weight"), b.raw("blk.0.ffn_up_exps.weight")[1:3])
        # a missing tensor is reported
        b.tensors.pop("blk.0.attn_q.weight")
        assert not spec.validate(b).ok


def test_convert_checkpoint_bf16_fp8_fp4_round_trips(capsys):
    from deepseek_v4_2080ti_b200.cli import convert_checkpoint as cc
    from deepseek_v4_2080ti_b200.formats import safetensors_io as sio
    torch.manual_seed(1)
    state = {"a.weight": (torch.randn(256, 256) * 0.05).bfloat16(), "b.weight": (torch.randn(128, 384) * 0.05).bfloat16(),
             "norm.weight": torch.ones(256).bfloat16(), "small.weight": torch.randn(8, 128).bfloat16()}
    with tempfile.TemporaryDirectory() as d:
        src, f8, f4, back = (os.path.join(d, n) for n in ("src", "fp8", "fp4", "back"))
        sio.write_checkpoint(src, iter(state.items()), config_json="{}")
        assert cc.main([src, f8, "--to", "fp8"]) == 0
        s8 = dict(sio.read_checkpoint(f8))
        assert s8["a.weight"].dtype == torch.float8_e4m3fn and s8["a.weight_scale_inv"].shape == (2, 2)
        assert s8["small.weight"].dtype == torch.bfloat16 and "norm.weight" in s8
        assert cc.main([f8, f4, "--to", "fp4", "--match", "a."]) == 0
        s4 = dict(sio.read_checkpoint(f4))
        assert s4["a.weight"].dtype == torch.uint8 and s4["a.scale"].shape == (256, 8) and s4["b.weight"].dtype == torch.float8_e4m3fn
        assert cc.main([f4, back, "--to", "bf16"]) == 0
        sb = dict(sio.read_checkpoint(back))
        assert sb["a.weight"].dtype == torch.bfloat16 and "a.scale" not in sb and "b.weight_scale_inv" not in sb
        err_b = (sb["b.weight"].float() - state["b.weight"].float()).norm() / state["b.weight"].float().norm()
        err_a = (sb["a.weight"].float() - state["a.weight"].float()).norm() / state["a.weight"].float().norm()
        assert err_b < 0.05 and err_a < 0.2
        assert os.path.exists(os.path.join(back, "config.json"))
        # NVFP4 as a target and as a source
        nv, back2 = os.path.join(d, "nvfp4"), os.path.join(d, "back2")
        assert cc.main([f8, nv, "--to", "nvfp4", "--match", "b."]) == 0
        sn = dict(sio.read_checkpoint(nv))
        assert sn["b.weight_packed"].shape == (128, 192) and sn["b.weight_scale"].dtype == torch.float8_e4m3fn
        assert sn["b.weight_global_scale"].numel() == 1 and "b.weight" not in sn and sn["a.weight"].dtype == torch.float8_e4m3fn
        assert cc.main([nv, back2, "--to", "bf16"]) == 0
        s2 = dict(sio.read_checkpoint(back2))
        err = (s2["b.weight"].float() - state["b.weight"].float()).norm() / state["b.weight"].float().norm()
        assert "b.weight_packed" not in s2 and err < 0.15
        # INT8 per-row (the host expert layout) as a target and as a source
        i8, back3 = os.path.join(d, "int8"), os.path.join(d, "back3")
        assert cc.main([f8, i8, "--to", "int8", "--match", "a."]) == 0
        si = dict(sio.read_checkpoint(i8))
        assert si["a.weight"].dtype == torch.int8 and si["a.scale"].shape == (256,) and si["a.scale"].dtype == torch.float32
        assert "a.weight_scale_inv" not in si and si["b.weight"].dtype == torch.float8_e4m3fn
        assert int(si["a.weight"].abs().max()) == 127
        assert cc.main([i8, back3, "--to", "bf16"]) == 0
        s3 = dict(sio.read_checkpoint(back3))
        err = (s3["a.weight"].float() - state["a.weight"].float()).norm() / state["a.weight"].float().norm()
        assert s3["a.weight"].dtype == torch.bfloat16 and "a.scale" not in s3 and err < 0.06


def test_inspect_safetensors_lists_filters_and_audits(capsys):
    from deepseek_v4_2080ti_b200.cli import inspect_safetensors as ins
    from deepseek_v4_2080ti_b200.formats import safetensors_io as sio
    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
    cfg = qh.QwenHybridConfig.tiny(layers=2)
    state = list(qh.synth_state(cfg, 0, "cpu", std=0.05))
    with tempfile.TemporaryDirectory() as d:
        sio.write_checkpoint(d, iter(state), shard_bytes=1 << 20, config_json=cfg.to_json())
        rep = ins.scan(d)
        assert len(rep["tensors"]) == len(state) and len(rep["shards"]) > 1 and "F8_E4M3" in rep["bytes_by_dtype"]
        assert rep["index"]["entries"] == len(state) and not rep["index"]["missing_from_shards"] and not rep["index"]["wrong_shard"]
        assert ins.main([d, "--grep", "layers.1.", "--audit", "--json"]) == 0
        out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
        assert out["audit"]["ok"] and all("layers.1." in t["name"] for t in out["tensors"]) and out["tensors"]
        assert ins.main([d, "--audit", "--tp-world", "3"]) == 3
        assert "audit_not_divisible=" in capsys.readouterr().out
    from deepseek_v4_2080ti_b200.cli import generate_glm, generate_gguf
    assert generate_glm.main is generate_gguf.main
