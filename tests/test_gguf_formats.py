"""GGUF block formats and container: dequantisers against the ``gguf`` Python package (independent oracle),
quantiser fidelity, writer -> reader round trip, stacked expert slicing, shard bundles."""
import os

import numpy as np
import pytest
import torch

from deepseek_v4_2080ti_b200.formats import gguf as G

TYPES = [G.GGMLType.Q8_0, G.GGMLType.Q4_K, G.GGMLType.Q5_K, G.GGMLType.Q2_K, G.GGMLType.IQ2_XXS, G.GGMLType.IQ3_XXS,
         G.GGMLType.IQ1_M, G.GGMLType.Q3_K, G.GGMLType.Q6_K, G.GGMLType.IQ2_XS, G.GGMLType.IQ4_XS]
# relative L2 error bounds for N(0, sigma) inputs (bits per weight: 8.5, 4.5, 5.5, 2.6, 2.06, 3.06, 1.75, 3.4, 6.6, 2.3, 4.25)
MAX_REL = {G.GGMLType.Q8_0: 0.01, G.GGMLType.Q4_K: 0.10, G.GGMLType.Q5_K: 0.05, G.GGMLType.Q2_K: 0.40,
           G.GGMLType.IQ2_XXS: 0.42, G.GGMLType.IQ3_XXS: 0.25, G.GGMLType.IQ1_M: 0.60, G.GGMLType.Q3_K: 0.22,
           G.GGMLType.Q6_K: 0.03, G.GGMLType.IQ2_XS: 0.36, G.GGMLType.IQ4_XS: 0.10}


@pytest.mark.parametrize("t", TYPES)
def test_dequantiser_matches_gguf_package_and_quantiser_tracks_input(t):
    gq = pytest.importorskip("gguf.quants")
    from gguf import GGMLQuantizationType
    torch.manual_seed(int(t))
    w = torch.randn(24, 768) * 0.02
    raw = G.quantize(w, t)
    assert raw.dtype == torch.uint8 and raw.shape == (24, 768 // G.BLOCK_ELEMS[t] * G.BLOCK_BYTES[t])
    ours = G.dequantize(raw, t, 768)
    oracle = torch.from_numpy(gq.dequantize(raw.numpy(), GGMLQuantizationType(int(t)))).float()
    assert torch.equal(ours, oracle)
    assert ((ours - w).norm() / w.norm()).item() < MAX_REL[t]
    # arbitrary (random) block bytes also decode identically: the dequantiser does not depend on our quantiser
    rnd = torch.randint(0, 256, raw.shape, dtype=torch.uint8, generator=torch.Generator().manual_seed(1))
    if t != G.GGMLType.Q8_0:
        # keep the fp16 scale fields finite
        nb = G.BLOCK_BYTES[t]
        r = rnd.view(24, -1, nb)
        for off in {G.GGMLType.Q4_K: (0, 2), G.GGMLType.Q5_K: (0, 2), G.GGMLType.Q2_K: (80, 82), G.GGMLType.IQ2_XXS: (0,),
                    G.GGMLType.IQ3_XXS: (0,), G.GGMLType.IQ1_M: (), G.GGMLType.Q3_K: (108,), G.GGMLType.Q6_K: (208,),
                    G.GGMLType.IQ2_XS: (0,), G.GGMLType.IQ4_XS: (0,)}[t]:
            r[..., off + 1] &= 0x3F
        if t == G.GGMLType.IQ1_M:
            r[..., 55] &= 0x3F                      # top nibble of the fp16 super-scale
    else:
        rnd.view(24, -1, 34)[..., 1] &= 0x3F
    a = G.dequantize(rnd, t, 768)
    b = torch.from_numpy(gq.dequantize(rnd.numpy(), GGMLQuantizationType(int(t)))).float()
    assert torch.equal(a, b)


def test_writer_reader_roundtrip_with_experts_and_metadata(tmp_path):
    torch.manual_seed(0)
    dense = torch.randn(64, 256) * 0.02
    experts = torch.randn(4, 32, 256) * 0.02
    raw_d = G.quantize(dense, G.GGMLType.Q4_K)
    raw_e = torch.stack([G.quantize(experts[e], G.GGMLType.IQ2_XXS) for e in range(4)])
    norm = torch.ones(256)
    meta = {"general.architecture": "minimax-m2", "general.name": "tiny", "minimax-m2.block_count": 2,
            "minimax-m2.rope.freq_base": 10000.0, "tokenizer.ggml.tokens": ["a", "b", "<eos>"],
            "tokenizer.ggml.token_type": [1, 1, 3], "tokenizer.ggml.eos_token_id": 2, "flag": True}
    path = str(tmp_path / "m.gguf")
    G.write_gguf(path, meta, [("blk.0.attn_q.weight", raw_d, G.GGMLType.Q4_K, (64, 256)),
                              ("blk.0.ffn_gate_exps.weight", raw_e, G.GGMLType.IQ2_XXS, (4, 32, 256)),
                              ("output_norm.weight", G.quantize(norm[None], G.GGMLType.F32), G.GGMLType.F32, (256,))])
    f = G.GGUFFile(path)
    assert f.metadata["general.architecture"] == "minimax-m2" and f.metadata["tokenizer.ggml.tokens"] == ["a", "b", "<eos>"]
    assert f.metadata["minimax-m2.block_count"] == 2 and f.metadata["flag"] is True
    assert abs(f.metadata["minimax-m2.rope.freq_base"] - 10000.0) < 1e-3
    ti = f.tensors["blk.0.ffn_gate_exps.weight"]
    assert ti.shape == (4, 32, 256) and ti.ggml_type == G.GGMLType.IQ2_XXS
    assert torch.equal(f.raw("blk.0.attn_q.weight"), raw_d)
    assert torch.equal(f.raw_expert("blk.0.ffn_gate_exps.weight", 2), raw_e[2])
    assert torch.equal(f.dequantized("blk.0.attn_q.weight"), G.dequantize(raw_d, G.GGMLType.Q4_K, 256))
    assert torch.equal(f.dequantized("output_norm.weight"), norm)
    # every tensor starts on the alignment boundary
    assert all((f.data_start + t.offset) % f.alignment == 0 for t in f.tensors.values())
    # the gguf package reads the same file
    rd = pytest.importorskip("gguf").GGUFReader(path)
    names = {t.name: t for t in rd.tensors}
    assert set(names) == set(f.tensors)
    assert np.array_equal(np.asarray(names["blk.0.attn_q.weight"].data).reshape(-1), raw_d.numpy().reshape(-1))


def test_shard_bundle(tmp_path):
    a = torch.randn(8, 32)
    for i, name in enumerate(["x", "y"], 1):
        G.write_gguf(str(tmp_path / f"model-{i:05d}-of-00002.gguf"),
                     {"general.architecture": "glm-dsa"} if i == 1 else {"split.no": i},
                     [(name, G.quantize(a * i, G.GGMLType.Q8_0), G.GGMLType.Q8_0, (8, 32))])
    b = G.read_bundle(str(tmp_path / "model-00002-of-00002.gguf"))
    assert b.architecture == "glm-dsa" and set(b.tensors) == {"x", "y"}
    assert torch.allclose(b.dequantized("y"), a * 2, atol=0.05)
    assert G.read_bundle(str(tmp_path)).architecture == "glm-dsa"
    os.remove(str(tmp_path / "model-00001-of-00002.gguf"))
    with pytest.raises(FileNotFoundError):
        G.read_bundle(str(tmp_path / "model-00002-of-00002.gguf"))
