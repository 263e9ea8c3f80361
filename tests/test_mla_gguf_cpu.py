"""GGUF checkpoints of the MLA + indexer MoE family (glm-dsa naming): metadata, name map, synthetic writer, raw-block
reader, registry validation and the inspection CLI - no GPU."""
import json
import os
import tempfile
from dataclasses import replace

import torch


def _cfg():
    from deepseek_v4_2080ti_b200.models import mla_moe as mm
    return replace(mm.MlaMoeConfig.tiny_cpu(), index_heads=4, index_dim=64, index_topk=16, first_dense_layers=1,
                   expert_format="bf16", mtp_layers=1, score_func="sigmoid", route_scale=2.5)


def test_metadata_roundtrip_and_layer_inventory():
    from deepseek_v4_2080ti_b200.models import mla_gguf as mg
    cfg = _cfg()
    assert mg.config_from_metadata(mg.metadata(cfg)) == cfg
    dense, moe, mtp = mg.layer_suffixes(cfg, 0), mg.layer_suffixes(cfg, 1), mg.layer_suffixes(cfg, cfg.num_layers)
    assert "ffn_gate.weight" in dense and "ffn_gate_exps.weight" not in dense
    assert {"ffn_gate_inp.weight", "exp_probs_b.bias", "ffn_down_exps.weight", "ffn_up_shexp.weight"} <= set(moe)
    assert "nextn.eh_proj.weight" in mtp and "nextn.eh_proj.weight" not in moe
    assert "indexer.proj.weight" in moe and "attn_k_b.weight" in moe
    no_q_lora = replace(cfg, q_lora_rank=0)
    assert "attn_q.weight" in mg.layer_suffixes(no_q_lora, 1) and "attn_q_a.weight" not in mg.layer_suffixes(no_q_lora, 1)


def test_raw_quant_slicing_keeps_blocks_whole():
    from deepseek_v4_2080ti_b200.formats import gguf as G
    from deepseek_v4_2080ti_b200.models.mla_gguf import RawQuant
    torch.manual_seed(0)
    w = torch.randn(12, 512) * 0.1
    rq = RawQuant(G.quantize(w, G.GGMLType.Q4_K), G.GGMLType.Q4_K, 12, 512)
    full = rq.dequant()
    assert torch.equal(rq.rows(3, 9).dequant(), full[3:9])
    assert torch.equal(rq.cols(256, 512).dequant(), full[:, 256:])
    assert rq.cols(128, 512) is None                       # would cut a 256-wide super-block
    other = RawQuant(G.quantize(w, G.GGMLType.Q8_0), G.GGMLType.Q8_0, 12, 512)
    assert RawQuant.cat([rq, other]) is None
    both = RawQuant.cat([rq.rows(0, 4), rq.rows(8, 12)])
    assert both.shape == (8, 512) and torch.equal(both.dequant(), torch.cat([full[:4], full[8:]]))


def test_written_checkpoint_reads_back_validates_and_inspects(capsys):
    from deepseek_v4_2080ti_b200.cli import inspect_gguf
    from deepseek_v4_2080ti_b200.formats import gguf as G
    from deepseek_v4_2080ti_b200.models import mla_gguf as mg
    from deepseek_v4_2080ti_b200.models import mla_moe as mm
    from deepseek_v4_2080ti_b200.models import registry
    from deepseek_v4_2080ti_b200.models.gqa_moe import TensorStore
    cfg = _cfg()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "glm.gguf")
        mg.write_synthetic_gguf(path, cfg, {"gate_up": "Q4_K", "down": "Q8_0"}, seed=3)
        b = G.read_bundle(path)
        assert b.tensors["blk.1.ffn_gate_exps.weight"].shape == (cfg.num_experts, cfg.expert_intermediate, cfg.hidden_size)
        assert b.tensors["blk.1.attn_k_b.weight"].shape == (cfg.num_heads, cfg.kv_lora_rank, cfg.qk_nope_dim)
        spec = registry.detect(b)
        assert spec.architecture == "glm-dsa" and "glm-dsa" in registry.architectures()
        rep = spec.validate(b)
        assert rep.ok and not rep.missing and not rep.unexpected and rep.routed_bytes > 0
        assert mg.config_from_metadata(b.metadata, b.tensors) == cfg
        got = dict(mg.read_state(TensorStore(b), cfg))
        want = dict(mm.synth_state(cfg, 3, "cpu", 0.02))
        assert set(got) == set(want)
        for k, v in want.items():
            g = got[k]
            is_raw = isinstance(g, mg.RawQuant)
            g = g.dequant() if is_raw else g.float()
            assert g.shape == v.shape, k
            err = ((g - v.float()).norm() / v.float().norm().clamp_min(1e-9)).item()
            assert err < (0.1 if is_raw or "wkv_b" in k or k == "embed.weight" else 1e-6), (k, err)
        assert isinstance(got["layers.1.ffn.experts.3.w2.weight"], mg.RawQuant)
        assert got["layers.1.ffn.experts.3.w2.weight"].t == G.GGMLType.Q8_0
        # a rank's view: only its experts and layers are touched
        part = dict(mg.read_state(TensorStore(b), cfg, expert_range=(2, 4), layer_range=(1, 2)))
        assert "layers.1.ffn.experts.2.w1.weight" in part and "layers.1.ffn.experts.4.w1.weight" not in part
        assert not any(k.startswith("layers.0.") for k in part) and "mtp.0.e_proj.weight" in part
        assert inspect_gguf.main([path, "--validate", "--placement", "--json"]) == 0
        out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
        assert out["architecture"] == "glm-dsa" and out["validation"]["ok"]
        # a missing tensor is reported by name
        tensors = [(n, b.raw(n), ti.ggml_type, tuple(ti.shape)) for n, ti in b.tensors.items() if n != "blk.1.exp_probs_b.bias"]
        bad = os.path.join(d, "bad.gguf")
        G.write_gguf(bad, b.metadata, tensors)
        rep = registry.detect(G.read_bundle(bad)).validate(G.read_bundle(bad))
        assert not rep.ok and rep.missing == ["blk.1.exp_probs_b.bias"]
