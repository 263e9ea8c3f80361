"""The Qwen-style MTP head in the fp32 CPU oracle: causal, recursive, and readable from bf16 or FP8 matrices."""
import torch

from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
from deepseek_v4_2080ti_b200.models.reference_cpu.qwen_hybrid_ref import QwenHybridRef, synth_mtp_state


def test_mtp_head_is_causal_recursive_and_format_agnostic():
    cfg = qh.QwenHybridConfig.tiny(layers=4)
    trunk = list(qh.synth_state(cfg, 0, "cpu", std=0.05))
    ref = QwenHybridRef(cfg, dict(trunk + synth_mtp_state(cfg, 0)))
    ids = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(2))
    logits = ref.forward(ids)
    hidden = ref.last_hidden
    assert hidden.shape == (12, cfg.hidden_size) and torch.allclose(hidden @ ref.p["lm_head.weight"].t(), logits)
    nxt = torch.cat([ids[1:], logits[-1:].argmax(-1)])          # the token after each position
    out, h1 = ref.mtp_forward(nxt, hidden)
    assert out.shape == (12, cfg.vocab_size) and h1.shape == hidden.shape and torch.isfinite(out).all()
    # causal: a prefix gives the same rows
    out8, _ = ref.mtp_forward(nxt[:8], hidden[:8])
    assert torch.allclose(out8, out[:8], atol=1e-5)
    # both inputs matter, and a second step consumes the head's own hidden
    assert (ref.mtp_forward(nxt.roll(1), hidden)[0] - out).abs().max() > 1e-3
    assert (ref.mtp_forward(nxt, hidden.roll(1, 0))[0] - out).abs().max() > 1e-3
    nxt2 = torch.cat([nxt[1:], out[-1:].argmax(-1)])
    out2, _ = ref.mtp_forward(nxt2, h1)
    assert out2.shape == out.shape and (out2 - out).abs().max() > 1e-3
    # FP8 block-scaled matrices of the same head stay close to the bf16 ones
    g = QwenHybridRef(cfg, dict(trunk + synth_mtp_state(cfg, 0, fp8_linears=True)))
    g.forward(ids)
    out_q, _ = g.mtp_forward(nxt, g.last_hidden)
    assert (out_q - out).abs().max() < 0.15 * out.abs().max()


def test_speculative_decoding_with_the_mtp_head_reproduces_greedy():
    from deepseek_v4_2080ti_b200.components.spec_gate import SpecGate
    from deepseek_v4_2080ti_b200.components.speculative import MtpDrafter, WholeSequenceTarget, speculative_generate
    cfg = qh.QwenHybridConfig.tiny(layers=4)
    ref = QwenHybridRef(cfg, dict(list(qh.synth_state(cfg, 0, "cpu", std=0.05)) + synth_mtp_state(cfg, 0)))
    prompt = torch.randint(0, cfg.vocab_size, (10,), generator=torch.Generator().manual_seed(4))
    ids, greedy = prompt.tolist(), []
    for _ in range(8):
        greedy.append(int(ref.forward(torch.tensor(ids))[-1].argmax()))
        ids.append(greedy[-1])
    tgt = WholeSequenceTarget(ref)
    out, st = speculative_generate(tgt, MtpDrafter(tgt), prompt, 8, block=2)
    assert out == greedy and st.rounds > 0 and st.accepted <= st.drafted <= 2 * st.rounds
    out_g, st_g = speculative_generate(tgt, MtpDrafter(tgt), prompt, 8, block=2, gate=SpecGate(2))
    assert out_g == greedy and st_g.gate["rounds"] >= 1
    # the first draft is the head's own prediction for the position after the committed token
    tgt.reset(); lg = tgt.forward(prompt)
    committed = int(lg[-1].argmax())
    d, conf = MtpDrafter(tgt).propose(prompt.tolist() + [committed], 2)
    want, _ = ref.mtp_forward(torch.tensor(prompt.tolist()[1:] + [committed]), tgt.hidden)
    assert d[0] == int(want[-1].argmax()) and len(conf) == 2 and all(c >= 0 for c in conf)
