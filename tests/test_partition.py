"""Partition policies: rule kinds by tensor name, per-rank slices, layer and expert ownership, key filtering."""
import pytest

from deepseek_v4_2080ti_b200.parallel import partition as pt


def test_rule_kinds():
    assert pt.rule_kind("layers.3.ffn.experts.17.w1.weight") == "expert_owned"
    assert pt.rule_kind("layers.3.ffn.shared_experts.w1.weight") == "column_parallel"
    assert pt.rule_kind("layers.3.ffn.shared_experts.w2.weight") == "row_parallel"
    assert pt.rule_kind("layers.0.attn.wo.weight") == "row_parallel" and pt.rule_kind("layers.0.attn.wq_b.weight") == "column_parallel"
    assert pt.rule_kind("layers.0.attn.wq_a.weight") == "replicated" and pt.rule_kind("layers.0.attn.indexer.wq_b.weight") == "replicated"
    assert pt.rule_kind("embed.weight") == "vocab_parallel" and pt.rule_kind("lm_head.weight") == "vocab_parallel"
    assert pt.rule_kind("model.language_model.layers.2.mlp.down_proj.weight_scale_inv") == "row_parallel"
    assert pt.rule_kind("model.language_model.layers.2.linear_attn.A_log") == "column_parallel"
    assert pt.rule_kind("layers.1.attn_norm.weight") == "replicated"
    assert pt.layer_of("model.language_model.layers.12.mlp.up_proj.weight") == 12 and pt.layer_of("norm.weight") is None
    assert pt.expert_of("layers.3.ffn.experts.17.w1.scale") == 17 and pt.expert_of("layers.3.ffn.shared_experts.w1.weight") is None


def test_tp_policy_slices_and_experts():
    p = pt.Partition("legacy", rank=3, world=4, n_layers=10, n_experts=64)
    assert p.policy == "tp" and p.layer_range == (0, 10) and p.expert_range == (48, 64)
    assert p.shard("layers.0.attn.wq_b.weight", (1024, 512)) == (0, 768, 256)
    assert p.shard("layers.0.attn.wo.weight", (512, 2048), block=128) == (1, 1536, 512)
    assert p.shard("layers.0.attn_norm.weight", (512,)) == (None, 0, 0)
    assert p.shard("embed.weight", (1001, 64)) == (0, 753, 248)                 # ragged vocabulary: last rank gets the rest
    assert p.shard("layers.1.linear_attn.A_log", (32,)) == (0, 24, 8)
    with pytest.raises(ValueError):
        p.shard("layers.0.attn.wo.weight", (512, 512), block=256)               # 128 columns per rank split a 256 block
    with pytest.raises(ValueError):
        p.shard("layers.0.attn.wq_b.weight", (1022, 512))
    assert p.owns("layers.9.ffn.experts.50.w1.weight") and not p.owns("layers.9.ffn.experts.3.w1.weight")
    assert p.owns("embed.weight") and p.owns("head.weight")
    with pytest.raises(ValueError):
        pt.Partition("tp", 0, 3, 4, n_experts=8)
    with pytest.raises(ValueError):
        pt.normalize_policy("diagonal")


def test_layer_pipeline_policy():
    ranks = [pt.Partition("layer_pp_4gpu", r, 8, n_layers=78, n_experts=256, stages=2) for r in range(8)]
    assert [p.layer_range for p in ranks] == [(0, 39)] * 4 + [(39, 78)] * 4
    assert ranks[5].expert_range == (64, 128) and ranks[5].layout.tp == 4
    assert ranks[0].owns("embed.weight") and not ranks[0].owns("head.weight") and not ranks[0].owns("norm.weight")
    assert ranks[4].owns("head.weight") and ranks[4].owns("mtp.0.e_proj.weight") and not ranks[4].owns("embed.weight")
    assert ranks[0].owns("layers.38.attn.wo.weight") and not ranks[0].owns("layers.39.attn.wo.weight")
    assert ranks[6].owns("layers.40.ffn.experts.130.w2.weight") and not ranks[6].owns("layers.40.ffn.experts.10.w2.weight")
    assert ranks[6].shard("layers.40.attn.wo.weight", (6144, 16384), 32) == (1, 8192, 4096)
    assert ranks[0].stage_of_layer(38) == 0 and ranks[0].stage_of_layer(39) == 1
    assert "stage=1/2" in ranks[7].describe() and "experts [192, 256)" in ranks[7].describe()
    # heavier early layers move the cut
    w = [3.0] * 3 + [1.0] * 7
    assert pt.Partition("layer_pp", 0, 2, 10, stages=2, layer_weights=w).layer_range == (0, 3)
