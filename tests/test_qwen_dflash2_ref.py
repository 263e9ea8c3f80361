"""The DFlash2 block-diffusion drafter for the Qwen hybrid target, fp32 on the host: dynamic grouped convolution,
windowed two-source attention, candidate selection (greedy chain and best path), refinement, checkpoint layout, and
the speculative loop."""
import itertools
import json

import pytest
import torch

from deepseek_v4_2080ti_b200.components.speculative import WholeSequenceTarget, speculative_generate
from deepseek_v4_2080ti_b200.formats import safetensors_io
from deepseek_v4_2080ti_b200.models import qwen_dflash2_ref as df
from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
from deepseek_v4_2080ti_b200.models.reference_cpu.qwen_hybrid_ref import QwenHybridRef


def _setup(seed=0, block=5, window=2048, **kw):
    cfg = qh.QwenHybridConfig.tiny(layers=4)
    ref = QwenHybridRef(cfg, dict(qh.synth_state(cfg, seed, "cpu", std=0.05)))
    dcfg = df.QwenDFlash2Config(hidden_size=cfg.hidden_size, intermediate_size=2 * cfg.hidden_size, vocab_size=cfg.vocab_size,
                                num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                                block_size=block, conv_group_size=16, conv_kernel_size=2, mask_token_id=cfg.vocab_size - 1,
                                selector_rank=8, selector_top_k=4, sliding_window=window, target_layer_ids=[1, 3])
    w = df.synth_dflash2_weights(dcfg, seed)
    dr = df.QwenDFlash2Ref(dcfg, w, ref.p["model.language_model.embed_tokens.weight"], ref.p["lm_head.weight"],
                           max_context=128, **kw)
    return cfg, ref, dcfg, w, dr


def test_dynamic_convolution_against_a_loop():
    g = torch.Generator().manual_seed(0)
    rows, h, gs, k = 5, 32, 8, 3
    x, dyn, base = torch.randn(rows, h, generator=g), torch.randn(rows, k * (h // gs), generator=g), torch.randn(k, h, generator=g)
    want = torch.zeros(rows, h)
    for r, c, t in itertools.product(range(rows), range(h), range(k)):
        if r - t >= 0:
            want[r, c] += x[r - t, c] * (base[t, c] + dyn[r, t * (h // gs) + c // gs])
    assert torch.allclose(df.dynamic_conv(x, dyn, base, gs), want, atol=1e-5)


def test_candidates_prefer_the_lower_token_on_ties_and_paths_agree_with_enumeration():
    logits = torch.tensor([[1.0, 3.0, 3.0, 0.5, 3.0], [0.0, 0.0, 2.0, 0.0, 0.0]])
    cand, val = df.top_candidates(logits, 3)
    assert cand.tolist() == [[1, 2, 4], [2, 0, 1]] and val[0].tolist() == [3.0, 3.0, 3.0]
    g = torch.Generator().manual_seed(2)
    rows, k, rank, vocab = 4, 3, 5, 11
    proj, unary = torch.randn(rows, rank, generator=g), torch.randn(rows, k, generator=g)
    pred, succ = torch.randn(vocab, rank, generator=g), torch.randn(vocab, rank, generator=g)
    cand = torch.stack([torch.randperm(vocab, generator=g)[:k] for _ in range(rows)])

    def score(path):                                            # path: one candidate index per row
        prev, s = 7, 0.0
        for r, j in enumerate(path):
            tok = int(cand[r, j])
            s += float(unary[r, j] + (pred[prev] * proj[r] * succ[tok]).sum())
            prev = tok
        return s
    best = max(itertools.product(range(k), repeat=rows), key=score)
    vit = df.select_path(proj, cand, unary, pred, succ, 7, viterbi=True)
    assert vit == [int(cand[r, j]) for r, j in enumerate(best)]
    greedy = df.select_path(proj, cand, unary, pred, succ, 7, viterbi=False)
    prev, want = 7, []
    for r in range(rows):
        sc = [float(unary[r, j] + (pred[prev] * proj[r] * succ[int(cand[r, j])]).sum()) for j in range(k)]
        prev = int(cand[r, max(range(k), key=lambda j: sc[j])])
        want.append(prev)
    assert greedy == want
    idx = lambda p: [cand[r].tolist().index(t) for r, t in enumerate(p)]
    assert score(idx(vit)) >= score(idx(greedy)) - 1e-6
    # one candidate per row: both selectors return it
    assert df.select_path(proj, cand[:, :1], unary[:, :1], pred, succ, 7, True) == cand[:, 0].tolist() \
        == df.select_path(proj, cand[:, :1], unary[:, :1], pred, succ, 7, False)


def test_context_is_prepared_lazily_and_the_window_limits_what_a_row_sees():
    cfg, ref, dcfg, w, dr = _setup()
    ids = torch.randint(0, cfg.vocab_size, (14,), generator=torch.Generator().manual_seed(1))
    ref.capture_layers = (1, 3)
    ref.forward(ids)
    taps = ref.last_taps
    dr.append_target_taps(taps[:6], 0)
    dr.append_target_taps(taps[6:], 6)
    assert dr.committed == 14 and dr.prepared == 0              # nothing projected yet
    one = dr.propose(5)
    assert dr.prepared == 14 and len(one.tokens) == dcfg.draft_tokens and one.candidates.shape == (4, 4)
    assert all(t in row for t, row in zip(one.tokens, one.candidates.tolist()))
    dr.crop_context(9)
    assert dr.prepared == 9
    short = dr.propose(5)
    fresh = _setup()[4]
    fresh.append_target_taps(taps[:9], 0)
    again = fresh.propose(5)
    assert short.tokens == again.tokens and torch.allclose(short.candidate_logits, again.candidate_logits, atol=1e-5)
    # a window of 3 keeps keys at distance < 3 only: a context row far behind no longer matters
    near = _setup(window=3)[4]
    near.append_target_taps(taps, 0)
    h1 = near.denoise([5] + [dcfg.mask_token_id] * 4)
    moved = taps.clone(); moved[:10] += 1.0                      # positions 0..9; row 0 sits at 14, sees 12 and 13 only
    far = _setup(window=3)[4]
    far.append_target_taps(moved, 0)
    assert torch.allclose(far.denoise([5] + [dcfg.mask_token_id] * 4), h1, atol=1e-6)
    wide = _setup(window=64)[4]
    wide.append_target_taps(moved, 0)
    ref_wide = _setup(window=64)[4]
    ref_wide.append_target_taps(taps, 0)
    assert (wide.denoise([5] + [dcfg.mask_token_id] * 4) - ref_wide.denoise([5] + [dcfg.mask_token_id] * 4)).abs().max() > 1e-4


def test_refinement_feeds_the_drafts_back_and_stops_at_a_fixed_point():
    cfg, ref, dcfg, w, dr = _setup(refine_passes=1)
    ids = torch.randint(0, cfg.vocab_size, (8,), generator=torch.Generator().manual_seed(3))
    ref.capture_layers = (1, 3)
    ref.forward(ids)
    dr.append_target_taps(ref.last_taps, 0)
    first = dr.propose(9)
    second, _, _ = dr._pass(9, [9] + first.tokens)
    dr.refine_passes = 2
    assert dr.propose(9).tokens == second
    dr.refine_passes = 6
    last = dr.propose(9).tokens
    assert len(last) == dcfg.draft_tokens
    dr.viterbi = True
    assert len(dr.propose(9).tokens) == dcfg.draft_tokens


def test_checkpoint_round_trip_and_validation(tmp_path):
    cfg, ref, dcfg, w, dr = _setup()
    (tmp_path / "config.json").write_text(json.dumps(dcfg.to_json()))
    safetensors_io.write_file(str(tmp_path / "model.safetensors"), w)
    cfg2, w2 = df.load_dflash2(tmp_path)
    assert cfg2 == dcfg and len(w2) == 6 + 15 * dcfg.num_hidden_layers and all(torch.equal(w[k], w2[k]) for k in w)
    # the full-size drafter holds 81 tensors
    full = df.QwenDFlash2Config(hidden_size=5120, intermediate_size=17408, vocab_size=248320, target_layer_ids=[5, 19, 33, 47, 61])
    assert len(df.expected_tensors(full)) == 81
    raw = dcfg.to_json(); raw["is_causal"] = True
    (tmp_path / "config.json").write_text(json.dumps(raw))
    with pytest.raises(ValueError, match="semantics"):
        df.load_dflash2(tmp_path)


@pytest.mark.parametrize("viterbi", [False, True])
def test_speculative_decoding_with_the_diffusion_drafter_reproduces_greedy(viterbi):
    cfg, ref, dcfg, w, dr = _setup(viterbi=viterbi)
    prompt = torch.randint(0, cfg.vocab_size, (10,), generator=torch.Generator().manual_seed(4))
    ids, greedy = prompt.tolist(), []
    for _ in range(9):
        greedy.append(int(ref.forward(torch.tensor(ids))[-1].argmax()))
        ids.append(greedy[-1])
    tgt = WholeSequenceTarget(ref)
    out, st = speculative_generate(tgt, df.QwenDFlash2Drafter(tgt, dr), prompt, 9, block=4)
    assert out == greedy and st.rounds > 0 and st.drafted <= 4 * st.rounds
