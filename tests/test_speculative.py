"""Host-side speculative decoding: the adaptive draft-length gate and the draft / verify / rollback loop."""
import pytest
import torch

from deepseek_v4_2080ti_b200.components.spec_gate import SpecCost, SpecGate
from deepseek_v4_2080ti_b200.components.speculative import PromptLookupDrafter, speculative_generate
from deepseek_v4_2080ti_b200.models import qwen4_exp_ref as q4


def test_gate_prior_keeps_the_full_block_and_learns_to_cut():
    g = SpecGate(4, SpecCost(plain_ms=300, draft_ms=200, verify_base_ms=300, verify_slope_ms=110))
    assert g.choose([0.0] * 4) == 4 and g.accept_prob(0.0) == pytest.approx(0.75)
    for _ in range(12):                                   # low-confidence positions keep failing, high ones pass
        g.observe([5.0, 5.0, -1.0, -1.0], accepted=2, drafted=4)
    assert g.accept_prob(5.0) > 0.95 and g.accept_prob(-1.0) < 0.2
    assert g.choose([5.0, 5.0, -1.0, -1.0]) == 2          # verify only what is likely to match
    assert g.choose([5.0] * 4) == 4
    assert g.choose([-1.0] * 4) == 0                      # a plain step beats a draft that will be thrown away
    s = g.stats()
    assert s["rounds"] == 12 and s["bucket_rates"]["[-inf,-0.5)"] == 0.0 and s["bucket_rates"]["[+3.0,+6.0)"] == 1.0


def test_gate_censors_positions_after_the_first_miss_and_forgets():
    g = SpecGate(3)
    g.observe([1.0, 2.0, 7.0], accepted=0, drafted=3)     # only position 0 is resolved
    assert g._seen[g.bucket(1.0)] == 1.0 and g._seen[g.bucket(2.0)] == 0.0 and g._seen[g.bucket(7.0)] == 0.0
    g.observe([1.0, 2.0, 7.0], accepted=3, drafted=3)
    assert g._seen[g.bucket(1.0)] == pytest.approx(1.9) and g._hit[g.bucket(7.0)] == 1.0
    g.observe([1.0], accepted=0, drafted=0)               # nothing verified, nothing learned
    assert g.rounds == 2
    g.note_skipped(); g.note_skipped(by_margin=True)
    assert (g.rounds, g.skipped, g.margin_skipped) == (4, 2, 1)
    with pytest.raises(ValueError):
        SpecGate(0)


def test_gate_margin_veto_min_draft_disabled_and_env(monkeypatch):
    g = SpecGate(4, margin_threshold=1.0)
    assert g.should_draft([5.0, 3.0]) and not g.should_draft([5.0, 4.5])
    assert SpecGate(4).should_draft([5.0, 4.99])
    off = SpecGate(4, enabled=False)
    assert off.choose([-9.0] * 4) == 4 and off.should_draft([0.0, 0.0])
    g2 = SpecGate(4, SpecCost(300, 50, 300, 110), min_draft=3)
    for _ in range(12):
        g2.observe([5.0, -1.0, -1.0, -1.0], accepted=1, drafted=4)
    assert g2.choose([5.0, -1.0, -1.0, -1.0]) == 3        # would cut to 1, floor is 3
    assert g2.choose([5.0, 5.0]) == 4                     # fewer scores than the block: no decision
    monkeypatch.setenv("POCKETLLM_SPEC_GATE", "1")
    monkeypatch.setenv("POCKETLLM_SPEC_GATE_PLAIN_MS", "5")
    monkeypatch.setenv("POCKETLLM_SPEC_GATE_MARGIN_THRESHOLD", "0.25")
    e = SpecGate.from_env(6)
    assert e.enabled and e.cost.plain_ms == 5.0 and e.margin_threshold == 0.25 and e.block == 6
    monkeypatch.delenv("POCKETLLM_SPEC_GATE")
    assert not SpecGate.from_env(6).enabled


def test_prompt_lookup_drafter():
    d = PromptLookupDrafter(3)
    toks, conf = d.propose([1, 2, 3, 4, 5, 9, 2, 3, 4], 3)
    assert toks == [5, 9, 2] and conf == [4.0] * 3        # matched the 3-gram (2, 3, 4)
    toks, conf = d.propose([7, 1, 8, 1], 2)
    assert toks == [8, 1] and conf == [0.0, 0.0]
    assert d.propose([1, 2, 3], 4) == ([], [])


class _Replay:
    """Target whose greedy continuation is a fixed cyclic sequence; counts passes and checks rollback discipline."""

    def __init__(self, seq, vocab=16):
        self.seq, self.vocab = seq, vocab
        self.reset()

    def reset(self):
        self.ctx = []

    def snapshot(self):
        return list(self.ctx)

    def restore(self, s):
        self.ctx = list(s)

    def forward(self, ids):
        rows = []
        for t in ids.reshape(-1).tolist():
            self.ctx.append(t)
            nxt = self.seq[len(self.ctx) % len(self.seq)]
            rows.append(torch.nn.functional.one_hot(torch.tensor(nxt), self.vocab).float() * 4)
        return torch.stack(rows)


def test_loop_equals_greedy_and_saves_passes_on_repetitive_text():
    seq = [3, 5, 7, 9, 11, 2]
    prompt = torch.tensor([seq[i % 6] for i in range(12)])
    tgt = _Replay(seq)
    tgt.reset(); lg = tgt.forward(prompt); greedy = []
    for _ in range(20):
        greedy.append(int(lg[-1].argmax())); lg = tgt.forward(torch.tensor([greedy[-1]]))
    out, st = speculative_generate(_Replay(seq), PromptLookupDrafter(3), prompt, 20, block=4)
    assert out == greedy and st.accepted == st.drafted > 0 and st.target_passes < 10 and st.replay_passes == 0
    # eos stops inside an accepted block
    out2, _ = speculative_generate(_Replay(seq), PromptLookupDrafter(3), prompt, 20, block=4, eos_token_id=greedy[2])
    assert out2 == greedy[:3]


def test_loop_on_the_recurrent_cpu_runtime_with_rollback_and_gate():
    cfg = q4.Qwen4ExpConfig()
    m = q4.Qwen4ExpRef(cfg, q4.synth_weights(cfg, 0), 160)
    g = torch.Generator().manual_seed(3)
    piece = torch.randint(1, cfg.vocab_size, (9,), generator=g)
    prompt = piece.repeat(4)
    greedy = m.generate(prompt, 14)
    out, st = speculative_generate(m, PromptLookupDrafter(3), prompt, 14, block=4)
    assert out == greedy and st.rounds > 0 and st.drafted >= st.accepted
    assert st.replay_passes <= st.rounds                  # a replay only after a miss
    gate = SpecGate(4, SpecCost(8, 1, 8, 0.3))
    out_g, st_g = speculative_generate(m, PromptLookupDrafter(3), prompt, 14, block=4, gate=gate)
    assert out_g == greedy and st_g.gate["rounds"] == gate.rounds
    # snapshot / restore is exact
    m.reset(); m.forward(prompt[:20]); snap = m.snapshot()
    a = m.forward(prompt[20:25]); m.restore(snap); b = m.forward(prompt[20:25])
    assert torch.equal(a, b)
