"""MoE model description read by the C++ core from GGUF metadata or from config.json
(csrc/core/model_config.cpp; reference: cpp_engine/core/model_config.cpp from_gguf / from_hf_config / to_string)."""
import json
import os
import subprocess

import pytest

cpp = pytest.importorskip("deepseek_v4_2080ti_b200.pocketllm_cpp")

V4_JSON = {
    "model_type": "deepseek_v4", "vocab_size": 129280, "hidden_size": 4096, "num_hidden_layers": 43,
    "num_attention_heads": 64, "num_key_value_heads": 1, "head_dim": 512, "q_lora_rank": 1024, "o_lora_rank": 1024,
    "o_groups": 8, "index_n_heads": 64, "index_head_dim": 128, "index_topk": 2048, "n_routed_experts": 256,
    "n_shared_experts": 1, "num_experts_per_tok": 6, "moe_intermediate_size": 2048, "routed_scaling_factor": 1.5,
    "swiglu_limit": 10.0, "max_position_embeddings": 1048576, "qk_rope_head_dim": 64, "rope_theta": 10000.0,
    "sliding_window": 128, "compress_rope_theta": 160000.0, "num_hash_layers": 3, "hc_mult": 4, "hc_sinkhorn_iters": 20,
    "compress_ratios": [0, 0] + [4, 128] * 20 + [4],
    "rope_scaling": {"type": "yarn", "factor": 16.0, "beta_fast": 32, "beta_slow": 1,
                     "original_max_position_embeddings": 65536},
}


def test_hf_json_fields_and_scaling_block():
    c = cpp.MoeModelConfig.from_hf_json_text(json.dumps(V4_JSON))
    j = json.loads(c.to_json_text())
    assert c.architecture == "deepseek_v4"
    assert (j["dim"], j["n_layers"], j["n_heads"], j["kv_heads"], j["head_dim"]) == (4096, 43, 64, 1, 512)
    assert (j["q_lora_rank"], j["o_lora_rank"], j["o_groups"]) == (1024, 1024, 8)
    assert (j["index_n_heads"], j["index_head_dim"], j["index_topk"]) == (64, 128, 2048)
    assert (j["n_routed_experts"], j["n_shared_experts"], j["n_activated_experts"], j["moe_inter_dim"]) == (256, 1, 6, 2048)
    assert j["route_scale"] == 1.5 and j["swiglu_limit"] == 10.0
    assert (j["rope_factor"], j["beta_fast"], j["beta_slow"], j["original_context_length"]) == (16.0, 32.0, 1.0, 65536)
    assert (j["window_size"], j["n_hash_layers"], j["hc_mult"], j["hc_sinkhorn_iters"]) == (128, 3, 4, 20)
    assert len(c.compress_ratios) == 43 and c.compress_ratios[2:4] == [4, 128]
    assert c.has_indexer and c.is_mla
    assert c.problems(tp_world=8, ep_world=8) == []
    text = c.describe()
    assert text.startswith("architecture=deepseek_v4 ") and " index_topk=2048" in text and "compress_ratios=0,0,4,128" in text
    assert " kv_lora_rank=" not in text          # unset fields are not printed


def test_short_spellings_and_text_config_wrapper():
    short = {"text_config": {"model_type": "glm_dsa", "vocab_size": 1000, "dim": 256, "n_layers": 4, "n_heads": 8,
                             "kv_lora_rank": 64, "qk_rope_head_dim": 16, "n_routed_experts": 16,
                             "n_activated_experts": 4, "moe_inter_dim": 128, "first_k_dense_replace": 1}}
    c = cpp.MoeModelConfig.from_hf_json_text(json.dumps(short))
    j = json.loads(c.to_json_text())
    assert c.architecture == "glm_dsa" and j["dim"] == 256 and j["n_dense_layers"] == 1 and j["kv_lora_rank"] == 64
    assert c.kv_bytes_per_token_layer == 2 * (64 + 16)
    with pytest.raises(RuntimeError):
        cpp.MoeModelConfig.from_hf_json_text("[1, 2]")


def test_problems_name_what_does_not_divide():
    bad = dict(V4_JSON, num_attention_heads=6, n_routed_experts=10, num_experts_per_tok=12, compress_ratios=[0, 4])
    c = cpp.MoeModelConfig.from_hf_json_text(json.dumps(bad))
    probs = " | ".join(c.problems(tp_world=4, ep_world=4))
    assert "n_heads 6 does not divide over 4" in probs
    assert "n_activated_experts must be in 1..n_routed_experts" in probs
    assert "n_routed_experts 10 does not divide over 4" in probs
    assert "compress_ratios has 2 entries for 43 layers" in probs
    empty = cpp.MoeModelConfig.from_hf_json_text("{}")
    assert any("dim is missing" in p for p in empty.problems())


def _write_gguf(path, arch, meta):
    from deepseek_v4_2080ti_b200.formats.gguf.writer import write_gguf
    full = {"general.architecture": arch}
    full.update(meta)
    write_gguf(str(path), full, [])


def test_gguf_metadata_with_prefix_fallbacks(tmp_path):
    p = tmp_path / "v4.gguf"
    _write_gguf(p, "deepseek4", {
        "deepseek4.embedding_length": 4096, "deepseek4.block_count": 43, "deepseek4.attention.head_count": 64,
        "deepseek4.attention.head_count_kv": 1, "deepseek4.attention.key_length": 512,
        "deepseek4.attention.indexer.head_count": 64, "deepseek4.attention.indexer.key_length": 128,
        "deepseek4.attention.indexer.top_k": 2048, "deepseek4.expert_count": 256, "deepseek4.expert_used_count": 6,
        "deepseek4.expert_feed_forward_length": 2048, "deepseek4.expert_weights_scale": 1.5,
        "deepseek4.rope.freq_base": 10000.0, "deepseek4.attention.sliding_window": 128,
        "deepseek4.hyper_connection.count": 4, "deepseek4.attention.compress_ratios": [0, 4, 128],
        "deepseek4.swiglu_clamp_exp": [7.0, 7.0, 10.0],
        "tokenizer.ggml.tokens": ["a", "b", "c", "d", "e"],
    })
    c = cpp.MoeModelConfig.from_gguf_file(str(p))
    j = json.loads(c.to_json_text())
    assert c.architecture == "deepseek4"
    assert j["vocab_size"] == 5                     # no vocab_size key: the token list's length
    assert (j["dim"], j["n_layers"], j["n_heads"], j["index_topk"], j["hc_mult"]) == (4096, 43, 64, 2048, 4)
    assert j["route_scale"] == 1.5 and c.compress_ratios == [0, 4, 128] and c.swiglu_clamp_exp == [7.0, 7.0, 10.0]
    # a file whose keys sit under an older prefix than its architecture string
    q = tmp_path / "old.gguf"
    _write_gguf(q, "minimax-m2", {"llama.embedding_length": 3072, "llama.block_count": 62,
                                  "minimax-m2.attention.head_count": 48, "llama.attention.head_count": 1,
                                  "llama.vocab_size": 200064, "minimax-m2.expert_count": 256,
                                  "minimax-m2.expert_used_count": 8, "minimax-m2.expert_feed_forward_length": 1536})
    d = cpp.MoeModelConfig.from_gguf(cpp.GGUFReader(str(q)))
    k = json.loads(d.to_json_text())
    assert (k["dim"], k["n_layers"], k["vocab_size"]) == (3072, 62, 200064)
    assert k["n_heads"] == 48                       # the architecture's own key wins over the fallback prefix
    assert d.problems(tp_world=8, ep_world=8) == []


def test_native_executable_describes_a_checkpoint(tmp_path):
    from deepseek_v4_2080ti_b200 import build
    exe = os.path.join(os.path.dirname(build.__file__), "bin", "pocketllm_engine")
    if not os.path.exists(exe):
        pytest.skip("native executable not built")
    (tmp_path / "config.json").write_text(json.dumps(V4_JSON))
    r = subprocess.run([exe, "--model-config", str(tmp_path), "--tp-world", "8", "--ep-world", "8"],
                       capture_output=True, text=True, timeout=60)
    assert r.returncode == 0, r.stderr
    assert "architecture=deepseek_v4" in r.stdout and "model_config_ok=1" in r.stdout and "indexer=1" in r.stdout
    r = subprocess.run([exe, "--model-config", str(tmp_path), "--tp-world", "7"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 3 and "problem: n_heads 64 does not divide over 7" in r.stdout
