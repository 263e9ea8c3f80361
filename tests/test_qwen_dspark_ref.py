"""The DSpark block drafter for the Qwen hybrid target, fp32 on the host: context memory from target taps, one-pass
block proposal with the bigram chain and the confidence read-out, checkpoint round trip, and the speculative loop."""
import json
import math

import pytest
import torch

from deepseek_v4_2080ti_b200.components.spec_gate import SpecGate
from deepseek_v4_2080ti_b200.components.speculative import WholeSequenceTarget, speculative_generate
from deepseek_v4_2080ti_b200.formats import safetensors_io
from deepseek_v4_2080ti_b200.models import qwen_dspark_ref as ds
from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
from deepseek_v4_2080ti_b200.models.reference_cpu.qwen_hybrid_ref import QwenHybridRef


def _setup(seed=0, block=4):
    cfg = qh.QwenHybridConfig.tiny(layers=4)
    ref = QwenHybridRef(cfg, dict(qh.synth_state(cfg, seed, "cpu", std=0.05)))
    dcfg = ds.QwenDSparkConfig(hidden_size=cfg.hidden_size, intermediate_size=2 * cfg.hidden_size, vocab_size=cfg.vocab_size,
                               num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                               block_size=block, mask_token_id=cfg.vocab_size - 1, markov_rank=16, target_layer_ids=[1, 3],
                               original_max_position_embeddings=64, rope_factor=4.0)
    w = ds.synth_dspark_weights(dcfg, seed)
    dr = ds.QwenDSparkRef(dcfg, w, ref.p["model.language_model.embed_tokens.weight"], ref.p["lm_head.weight"], max_context=128)
    return cfg, ref, dcfg, w, dr


def test_yarn_frequencies_keep_fast_pairs_and_stretch_slow_ones():
    cfg = ds.QwenDSparkConfig(hidden_size=64, intermediate_size=64, vocab_size=32, head_dim=128, target_layer_ids=[0])
    inv = ds.yarn_inv_freqs(cfg).double()
    plain = 1.0 / (cfg.rope_theta ** (torch.arange(0, 128, 2, dtype=torch.float64) / 128))
    ratio = plain / inv
    assert torch.allclose(ratio[:4], torch.ones(4, dtype=torch.float64), rtol=1e-5)       # fast pairs untouched
    assert torch.allclose(ratio[-4:], torch.full((4,), 32.0, dtype=torch.float64), rtol=1e-5)   # slow pairs / factor
    assert (ratio[1:] >= ratio[:-1] * (1 - 1e-5)).all()                                        # a monotone ramp in between
    assert cfg.attention_factor == pytest.approx(0.1 * math.log(32.0) + 1.0)


def test_context_memory_is_incremental_and_crop_restores_it():
    cfg, ref, dcfg, w, dr = _setup()
    ids = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(1))
    ref.capture_layers = (1, 3)
    ref.forward(ids)
    taps = ref.last_taps
    assert taps.shape == (12, 2 * cfg.hidden_size)
    dr.append_target_taps(taps, 0)
    one = dr.propose(5)
    k_all = [k[:12].clone() for k in dr.ctx_k]
    dr.reset()
    dr.append_target_taps(taps[:7], 0)
    dr.append_target_taps(taps[7:], 7)
    assert all(torch.allclose(a, k[:12], atol=1e-6) for a, k in zip(k_all, dr.ctx_k))
    two = dr.propose(5)
    assert two.tokens == one.tokens and two.confidences == pytest.approx(one.confidences, abs=1e-5)
    # proposing does not change the committed context; cropping forgets the tail
    assert dr.committed == 12
    dr.crop_context(7)
    short = dr.propose(5)
    dr.reset(); dr.append_target_taps(taps[:7], 0)
    again = dr.propose(5)
    assert short.tokens == again.tokens and short.top_logits == pytest.approx(again.top_logits, abs=1e-5)
    with pytest.raises(ValueError):
        dr.append_target_taps(taps[:2], 3)                     # must continue at the committed position
    with pytest.raises(ValueError):
        dr.crop_context(9)


def test_block_rows_see_each_other_and_the_bigram_chain_is_sequential():
    cfg, ref, dcfg, w, dr = _setup()
    ids = torch.randint(0, cfg.vocab_size, (9,), generator=torch.Generator().manual_seed(3))
    ref.capture_layers = (1, 3)
    ref.forward(ids)
    dr.append_target_taps(ref.last_taps, 0)
    x = dr.block_hidden(7)
    assert x.shape == (dcfg.block_size, cfg.hidden_size) and torch.isfinite(x).all()
    # no causal mask inside the block: another anchor changes every row, the mask rows included
    y = dr.block_hidden(8)
    assert ((x - y).abs().amax(-1) > 1e-4).all()
    # the chain by hand
    prop = dr.propose(7)
    base = x @ dr.head.t()
    prev, toks, emb = 7, [], []
    for r in range(dcfg.block_size):
        e = dr.w["markov_head.markov_w1.weight"][prev]
        emb.append(e)
        prev = int((base[r] + dr.w["markov_head.markov_w2.weight"] @ e).argmax())
        toks.append(prev)
    assert prop.tokens == toks
    conf = torch.sigmoid(torch.cat([x, torch.stack(emb)], -1) @ dr.w["confidence_head.proj.weight"][0]
                         + dr.w["confidence_head.proj.bias"][0])
    assert prop.confidences == pytest.approx(conf.tolist(), abs=1e-6) and all(0.0 < c < 1.0 for c in prop.confidences)
    # the bias matters: without it at least one row of this seed picks another token
    assert toks != base.argmax(-1).tolist()
    # the context matters
    dr.crop_context(4)
    assert (dr.block_hidden(7) - x).abs().max() > 1e-4


def test_checkpoint_round_trip_and_validation(tmp_path):
    cfg, ref, dcfg, w, dr = _setup()
    (tmp_path / "config.json").write_text(json.dumps(dcfg.to_json()))
    safetensors_io.write_file(str(tmp_path / "model.safetensors"), w)
    cfg2, w2 = ds.load_dspark(tmp_path)
    assert cfg2 == dcfg and set(w2) == set(w) and len(w2) == 7 + 11 * dcfg.num_hidden_layers
    assert all(torch.equal(w[k], w2[k]) for k in w)
    bad = dict(w); bad.pop("norm.weight")
    (tmp_path / "b").mkdir()
    (tmp_path / "b" / "config.json").write_text(json.dumps(dcfg.to_json()))
    safetensors_io.write_file(str(tmp_path / "b" / "model.safetensors"), bad)
    with pytest.raises(ValueError, match="norm.weight"):
        ds.load_dspark(tmp_path / "b")
    raw = dcfg.to_json(); raw["markov_head_type"] = "gated"
    (tmp_path / "b" / "config.json").write_text(json.dumps(raw))
    with pytest.raises(ValueError, match="markov_head_type"):
        ds.load_dspark(tmp_path / "b")


def test_speculative_decoding_with_the_block_drafter_reproduces_greedy():
    cfg, ref, dcfg, w, dr = _setup(block=4)
    prompt = torch.randint(0, cfg.vocab_size, (10,), generator=torch.Generator().manual_seed(4))
    ids, greedy = prompt.tolist(), []
    for _ in range(10):
        greedy.append(int(ref.forward(torch.tensor(ids))[-1].argmax()))
        ids.append(greedy[-1])
    tgt = WholeSequenceTarget(ref)
    out, st = speculative_generate(tgt, ds.QwenDSparkDrafter(tgt, dr), prompt, 10, block=4)
    assert out == greedy and st.rounds > 0 and st.accepted <= st.drafted <= 4 * st.rounds
    assert dr.committed <= len(prompt) + 10
    # a second sequence through the same drafter starts from an empty context
    prompt2 = torch.randint(0, cfg.vocab_size, (6,), generator=torch.Generator().manual_seed(5))
    ids, greedy2 = prompt2.tolist(), []
    for _ in range(6):
        greedy2.append(int(ref.forward(torch.tensor(ids))[-1].argmax()))
        ids.append(greedy2[-1])
    out2, _ = speculative_generate(tgt, ds.QwenDSparkDrafter(tgt, dr), prompt2, 6, block=4, gate=SpecGate(4))
    assert out2 == greedy2


def test_a_drafter_that_agrees_with_the_target_is_accepted_whole():
    """With the bigram tables replaced by the target's own next-token table (a target that only looks at the previous
    token is imitated exactly), every proposed token is accepted: the loop's accounting of full blocks."""
    cfg, ref, dcfg, w, dr = _setup(block=3)
    prompt = torch.randint(0, cfg.vocab_size, (8,), generator=torch.Generator().manual_seed(6))
    tgt = WholeSequenceTarget(ref)

    class Oracle:                                              # proposes what the target would say
        def propose(self, context, k):
            ids, out = list(context), []
            for _ in range(k):
                out.append(int(ref.forward(torch.tensor(ids))[-1].argmax()))
                ids.append(out[-1])
            return out, [1.0] * k
    out, st = speculative_generate(tgt, Oracle(), prompt, 9, block=3)
    assert st.accepted == st.drafted and st.replay_passes == 0 and len(out) == 9
