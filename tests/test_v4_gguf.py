"""DeepSeek-V4 GGUF checkpoints: name table, metadata round trip, validation report, and loading into the fp32 block
runtime (models/v4_gguf.py; reference: src/loader/mappings/deepseek_v4.py build_ds4_tensor_mappings / validation)."""
import pytest
import torch

from deepseek_v4_2080ti_b200.formats import gguf as G
from deepseek_v4_2080ti_b200.models import v4_gguf
from deepseek_v4_2080ti_b200.models.v4_block_ref import V4BlockRef, V4Config, synth_weights


def _cfg():
    return V4Config(vocab_size=96, dim=64, n_layers=3, compress_ratios=(0, 4, 8), n_hash_layers=1, moe_inter=32)


def test_table_covers_the_runtime_weights_exactly():
    cfg = _cfg()
    w = synth_weights(cfg)
    entries = v4_gguf.expected_entries(cfg)
    keys = [e.key for e in entries]
    assert len(keys) == len(set(keys))
    assert set(keys) == set(w)                      # nothing the runtime needs is unnamed, nothing is named twice
    names = {e.gguf for e in entries}
    assert "blk.0.ffn_gate_tid2eid.weight" in names and "blk.0.exp_probs_b.bias" not in names      # hash layer
    assert "blk.1.exp_probs_b.bias" in names and "blk.1.indexer.attn_q_b.weight" in names           # ratio 4: indexer
    assert "blk.2.attn_compressor_kv.weight" in names and "blk.2.indexer.proj.weight" not in names  # ratio 8: no indexer
    assert "blk.0.attn_compressor_ape.weight" not in names                                          # window-only layer
    assert "blk.3.nextn.e_proj.weight" in names                                                     # MTP block after the last layer
    stacked = [e for e in entries if e.gguf == "blk.1.ffn_up_exps.weight"]
    assert [e.expert for e in stacked] == list(range(cfg.n_experts)) and stacked[2].key == "layers.1.ffn.experts.2.w3"


def test_metadata_round_trip():
    cfg = _cfg()
    md = v4_gguf.metadata(cfg)
    assert md["general.architecture"] == "deepseek4" and md["deepseek4.attention.compress_ratios"] == [0, 4, 8]
    assert v4_gguf.config_from_metadata(md) == cfg
    with pytest.raises(ValueError):
        v4_gguf.config_from_metadata({"general.architecture": "llama"})
    bad = dict(md)
    del bad["deepseek4.expert_count"]
    with pytest.raises(KeyError, match="expert_count"):
        v4_gguf.config_from_metadata(bad)


def test_fp32_file_reproduces_the_runtime_bit_for_bit(tmp_path):
    cfg = _cfg()
    w = synth_weights(cfg, seed=3)
    path = str(tmp_path / "v4.gguf")
    v4_gguf.write_gguf(path, cfg, w, "F32")
    cfg2, w2 = v4_gguf.load(path)
    assert cfg2 == cfg and set(w2) == set(w)
    for k in w:
        assert w2[k].shape == w[k].shape, k
        assert torch.equal(w2[k].to(w[k].dtype), w[k]), k
    prompt = torch.arange(5, 25) % cfg.vocab_size
    assert V4BlockRef(cfg2, w2).generate(prompt, 6) == V4BlockRef(cfg, w).generate(prompt, 6)


def test_q8_0_file_loads_with_quantisation_error_only(tmp_path):
    cfg = _cfg()
    w = synth_weights(cfg, seed=4)
    path = str(tmp_path / "v4q.gguf")
    v4_gguf.write_gguf(path, cfg, w, "Q8_0")
    b = G.read_bundle(path)
    assert b.tensors["blk.1.ffn_gate_exps.weight"].ggml_type == G.GGMLType.Q8_0
    assert b.tensors["blk.1.ffn_gate_exps.weight"].shape == (cfg.n_experts, cfg.moe_inter, cfg.dim)
    assert b.tensors["blk.1.attn_compressor_ape.weight"].ggml_type in (G.GGMLType.Q8_0, G.GGMLType.F16)
    assert b.tensors["output_norm.weight"].ggml_type == G.GGMLType.F32
    _, w2 = v4_gguf.load(path)
    for k in ("layers.1.attn.wq_b", "layers.2.ffn.experts.3.w2", "embed"):
        rel = (w2[k] - w[k]).norm() / w[k].norm()
        assert rel < 1e-2, (k, float(rel))
    assert torch.equal(w2["layers.0.ffn.tid2eid"], w["layers.0.ffn.tid2eid"])
    logits = V4BlockRef(cfg, w2).forward(torch.arange(12) % cfg.vocab_size)
    assert torch.isfinite(logits).all()


def test_validation_lists_every_problem(tmp_path):
    cfg = _cfg()
    w = synth_weights(cfg, seed=5)

    class T:
        def __init__(self, shape):
            self.shape = shape

    good = {}
    for e in v4_gguf.expected_entries(cfg):
        s = tuple(w[e.key].shape)
        good[e.gguf] = T((cfg.n_experts, *s) if e.kind == "experts" else s)
    assert v4_gguf.validate(good, cfg).ok
    bad = dict(good)
    del bad["blk.1.attn_q_b.weight"]
    bad["blk.2.ffn_norm.weight"] = T((cfg.dim + 1,))
    bad["blk.0.something_new.weight"] = T((4, 4))
    v = v4_gguf.validate(bad, cfg)
    assert not v.ok
    assert v.missing == ["blk.1.attn_q_b.weight"] and v.unmapped == ["blk.0.something_new.weight"]
    assert len(v.shape_errors) == 1 and "blk.2.ffn_norm.weight" in v.shape_errors[0] and "layers.2.ffn_norm" in v.shape_errors[0]
    # a file with a missing tensor refuses to load, naming it
    path = str(tmp_path / "broken.gguf")
    v4_gguf.write_gguf(path, cfg, w, "F32")
    import deepseek_v4_2080ti_b200.models.v4_gguf as m
    rows = m.LAYER_ROWS
    try:
        m.LAYER_ROWS = rows + (m.Row("blk.{L}.extra.weight", "{P}extra", "vector"),)
        with pytest.raises(ValueError, match="missing blk.0.extra.weight"):
            m.load(path)
    finally:
        m.LAYER_ROWS = rows


def test_registered_family_validates_and_generates(tmp_path):
    from deepseek_v4_2080ti_b200.models import registry
    cfg = _cfg()
    w = synth_weights(cfg, seed=6)
    path = str(tmp_path / "v4r.gguf")
    v4_gguf.write_gguf(path, cfg, w, "F32")
    b = G.read_bundle(path)
    spec = registry.detect(b)
    assert spec.architecture == "deepseek4" and "deepseek4" in registry.architectures()
    rep = spec.validate(b)
    assert rep.ok and not rep.missing and not rep.unexpected, (rep.missing[:3], rep.unexpected[:3], rep.unsupported)
    assert rep.routed_bytes > 0 and rep.total_bytes > rep.routed_bytes
    _, rt = spec.build_runtime(b, "cpu")
    prompt = torch.arange(3, 19, dtype=torch.int32) % cfg.vocab_size
    slot = rt.allocate()
    tok = rt.prefill(slot, prompt)
    out = [int(tok)]
    for _ in range(4):
        tok = rt.decode([slot], tok.to(torch.int32))
        out.append(int(tok))
    assert out == V4BlockRef(cfg, w).generate(prompt, 5)
    with pytest.raises(ValueError):
        spec.build_runtime(b, "cpu", 0, 2)


def test_gguf_cli_serves_the_host_family_without_a_gpu(tmp_path):
    import subprocess
    import sys
    cfg = _cfg()
    w = synth_weights(cfg, seed=7)
    path = str(tmp_path / "v4c.gguf")
    v4_gguf.write_gguf(path, cfg, w, "F32")
    r = subprocess.run([sys.executable, "-m", "deepseek_v4_2080ti_b200.cli.generate_gguf", "--gguf", path,
                        "--token-ids", "3,4,5,6,7,8", "--max-new-tokens", "4"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-800:]
    want = V4BlockRef(cfg, w).generate(torch.tensor([3, 4, 5, 6, 7, 8]), 4)
    assert "tokens=" + ",".join(map(str, want)) in r.stdout and "family=deepseek4" in r.stdout


def test_long_context_options_of_the_registered_family(tmp_path, monkeypatch):
    """The host pool alone leaves the tokens unchanged; a retriever checkpoint is read, checked and used."""
    from deepseek_v4_2080ti_b200.formats import safetensors_io
    from deepseek_v4_2080ti_b200.models import registry
    from deepseek_v4_2080ti_b200.models import v4_flashmemory as lc
    cfg = _cfg()
    w = synth_weights(cfg, seed=8)
    path = str(tmp_path / "v4l.gguf")
    v4_gguf.write_gguf(path, cfg, w, "F32")
    b = G.read_bundle(path)
    spec = registry.detect(b)
    prompt = torch.arange(3, 27, dtype=torch.int32) % cfg.vocab_size

    def run(rt, n=6):
        slot = rt.allocate()
        tok = rt.prefill(slot, prompt)
        out = [int(tok)]
        for _ in range(n - 1):
            tok = rt.decode([slot], tok.to(torch.int32))
            out.append(int(tok))
        return out
    want = V4BlockRef(cfg, w).generate(prompt, 6)
    _, rt = spec.build_runtime(b, "cpu", kv_swap_chunks=max(cfg.index_topk, 4), kv_swap_chunk_entries=2)
    assert isinstance(rt.rt, lc.V4LongContextRuntime) and run(rt) == want and rt.rt.swap_stats()["d2h_bytes"] > 0
    monkeypatch.setenv("POCKETLLM_GGUF_KV_SWAP", "1")
    monkeypatch.setenv("POCKETLLM_GGUF_KV_SWAP_GPU_CHUNKS", "64")
    _, rt = spec.build_runtime(b, "cpu")
    assert isinstance(rt.rt, lc.V4LongContextRuntime) and run(rt) == want
    monkeypatch.delenv("POCKETLLM_GGUF_KV_SWAP")
    ck = str(tmp_path / "flashmemory.safetensors")
    rw = lc.synth_retriever_weights(cfg, n_retrievers=2, seed=4)
    safetensors_io.write_file(ck, {k: v.to(torch.bfloat16) for k, v in rw.items()})
    got = lc.load_retrievers(ck, cfg.dim)
    assert set(got) == set(rw) and all(v.dtype == torch.float32 for v in got.values())
    _, rt = spec.build_runtime(b, "cpu", flashmemory=ck, flashmemory_ensemble="mean")
    out = run(rt)
    assert len(out) == 6 and rt.rt.retriever is not None and rt.rt.last_selection is not None and not rt.rt.retriever.use_max
    del rw["retrievers.l1.q_norm_weight"]
    safetensors_io.write_file(ck, rw)
    with pytest.raises(ValueError, match="missing retrievers.l1.q_norm_weight"):
        spec.build_runtime(b, "cpu", flashmemory=ck)
    safetensors_io.write_file(ck, lc.synth_retriever_weights(cfg, n_retrievers=1, seed=4))
    with pytest.raises(ValueError, match="does not fit a model of width"):
        lc.load_retrievers(ck, cfg.dim + 16)


def test_block_drafter_in_front_of_the_registered_family(tmp_path):
    from deepseek_v4_2080ti_b200.formats import safetensors_io
    from deepseek_v4_2080ti_b200.models import registry, v4_dspark_ref as vd
    cfg = _cfg()
    w = synth_weights(cfg, seed=9)
    path = str(tmp_path / "v4s.gguf")
    v4_gguf.write_gguf(path, cfg, w, "F32")
    b = G.read_bundle(path)
    spec = registry.detect(b)
    prompt = torch.arange(5, 21, dtype=torch.int32) % cfg.vocab_size
    want = V4BlockRef(cfg, w).generate(prompt, 9)

    def run(rt, n=9):
        slot = rt.allocate()
        tok = rt.prefill(slot, prompt)
        out = [int(tok)]
        for _ in range(n - 1):
            tok = rt.decode([slot], tok.to(torch.int32))
            out.append(int(tok))
        return out
    _, rt = spec.build_runtime(b, "cpu", dspark="synthetic", dspark_block=3)
    assert run(rt) == want and rt.stats()["spec_rounds"] > 0 and rt.stats()["spec_drafted"] >= rt.stats()["spec_accepted"]
    assert run(rt) == want                                           # a second sequence on the same adapter
    layer_ids = (0, cfg.n_layers - 1)
    dw = vd.synth_dspark_weights(cfg, n_stages=1, n_target=2, seed=4)
    ck = str(tmp_path / "dspark.safetensors")
    vd.save_dspark_weights(ck, dw, layer_ids)
    back, ids = vd.load_dspark_weights(ck, cfg)
    assert ids == layer_ids and set(back) == set(dw)
    _, rt = spec.build_runtime(b, "cpu", dspark=ck, spec_gate="1")
    assert run(rt) == want
    with pytest.raises(ValueError, match="does not match"):
        spec.build_runtime(b, "cpu", dspark=ck, dspark_target_layers="0")


def test_public_api_serves_the_host_family_with_its_options(tmp_path):
    from pocketllm import LLM, ConfigurationError, EngineArgs, SamplingParams
    cfg = _cfg()
    w = synth_weights(cfg, seed=7)
    path = str(tmp_path / "v4api.gguf")
    v4_gguf.write_gguf(path, cfg, w, "F32")
    prompt = [3, 4, 5, 6, 7, 8]
    want = V4BlockRef(cfg, w).generate(torch.tensor(prompt), 6)
    for opts, key in (({}, None), ({"dspark": "synthetic", "dspark_block": 3}, "spec_rounds"),
                      ({"kv_swap_chunks": 8, "kv_swap_chunk_entries": 2}, "kv_swap_d2h_bytes")):
        llm = LLM(EngineArgs(model=path, device="cpu", max_model_len=64, backend_options=opts))
        res = llm.generate([{"prompt_token_ids": prompt}], SamplingParams(max_tokens=6))[0]
        assert res.token_ids == want, opts
        if key:                                               # the pool's counters restart with every sequence
            assert key in llm.health().details and (key.startswith("kv_swap") or llm.health().details[key] > 0)
        with pytest.raises(ConfigurationError, match="not a token id"):
            llm.generate([{"prompt_token_ids": [cfg.vocab_size]}], SamplingParams(max_tokens=1))
        llm.close()
