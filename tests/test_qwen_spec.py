"""Speculative decoding on the Qwen-style hybrid GPU runtime: the output must be token for token the plain greedy
output, whatever the drafts are (multi-token-prediction head, prompt lookup, perfect or deliberately wrong drafts that
exercise the recurrent-state rollback at every row), and the head's hidden states must match the fp32 oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _model(layers=4, seed=0):
    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
    from deepseek_v4_2080ti_b200.models.reference_cpu.qwen_hybrid_ref import synth_mtp_state
    cfg = qh.QwenHybridConfig.tiny(layers=layers)
    state = list(qh.synth_state(cfg, seed, "cuda", std=0.05)) + \
        [(n, t.cuda()) for n, t in synth_mtp_state(cfg, seed, std=0.05, fp8_linears=True)]
    w = qh.QwenHybridWeights(cfg, iter(state), "cuda")
    assert w.mtp is not None
    rt = qh.QwenHybridRuntime(cfg, w, max_slots=2, max_context=640)
    return cfg, state, rt


@pytest.mark.parametrize("method,k", [("mtp", 1), ("mtp", 2), ("mtp", 3), ("ngram", 3)])
def test_speculative_output_equals_greedy(method, k):
    from deepseek_v4_2080ti_b200.models.qwen_spec import QwenSpeculator
    from deepseek_v4_2080ti_b200.ops import _lib
    cfg, _, rt = _model()
    torch.manual_seed(5)
    prompt = torch.randint(0, cfg.vocab_size, (150,), dtype=torch.int32)
    # the plain greedy output per prefill chunking (a different chunking rounds differently, so near-ties may flip)
    plain = {chunk: rt.generate(prompt, 40, chunk=chunk) for chunk in (8192, 64)}
    spec = QwenSpeculator(rt, k=k, method=method)
    for chunk in (8192, 64):                       # one-chunk and chunked prefill (the head follows every chunk)
        greedy = plain[chunk]
        out = spec.generate(prompt, 40, chunk=chunk)
        torch.cuda.synchronize()
        _lib.check_status()
        assert out == greedy, (method, k, chunk, out, greedy)
    s = spec.stats
    assert s.rounds + s.plain_steps > 0 and s.accepted <= s.drafted
    rt.keep_hidden = False
    assert rt.generate(prompt, 40) == plain[8192]  # the runtime is left in a usable state


@pytest.mark.parametrize("k,wrong_at", [(3, None), (3, 0), (3, 1), (3, 2), (1, 0), (5, 3)])
def test_given_drafts_accept_and_rollback_at_every_row(k, wrong_at):
    """Drafts taken from the known greedy continuation are all accepted (K+1 tokens per pass); a wrong token at row
    ``wrong_at`` cuts the block there and the recurrent state is restored from that row's checkpoint."""
    from deepseek_v4_2080ti_b200.models.qwen_spec import QwenSpeculator
    cfg, _, rt = _model()
    torch.manual_seed(6)
    prompt = torch.randint(0, cfg.vocab_size, (97,), dtype=torch.int32)
    n_new = 31
    greedy = rt.generate(prompt, n_new + 8)

    class Given(QwenSpeculator):
        def _propose(self, slot):
            done = len(self.seqs[slot].history) - prompt.numel()      # tokens generated so far (incl. committed)
            d = list(greedy[done:done + self.k])
            if wrong_at is not None and wrong_at < len(d):
                d[wrong_at] = (d[wrong_at] + 1) % cfg.vocab_size
            return torch.tensor(d, dtype=torch.int32, device="cuda")

    spec = Given(rt, k=k, method="ngram")
    out = spec.generate(prompt, n_new)
    assert out == greedy[:n_new], (out, greedy[:n_new])
    s = spec.stats
    if wrong_at is None:
        assert s.accepted == s.drafted and s.rollbacks == 0 and s.tokens_per_pass == k + 1
    else:
        assert s.rollbacks == s.rounds and s.accepted == wrong_at * s.rounds


def test_head_hidden_states_match_the_fp32_oracle():
    from deepseek_v4_2080ti_b200.models.qwen_spec import QwenSpeculator
    from deepseek_v4_2080ti_b200.models.reference_cpu.qwen_hybrid_ref import QwenHybridRef
    cfg, state, rt = _model(layers=2)
    torch.manual_seed(7)
    prompt = torch.randint(0, cfg.vocab_size, (48,), dtype=torch.int32)
    ref = QwenHybridRef(cfg, [(n, t.cpu()) for n, t in state])
    logits = ref.forward(prompt)
    t0 = int(logits[-1].argmax())
    nxt = torch.cat([prompt[1:], torch.tensor([t0], dtype=torch.int32)])
    _, want = ref.mtp_forward(nxt, ref.last_hidden)
    spec = QwenSpeculator(rt, k=1, method="mtp")
    slot = spec.allocate()
    first = spec.prefill(slot, prompt.cuda())
    assert first == t0
    st = rt.seqs[slot]
    # run the head once more over the prompt rows (rewrites the same cache rows) to read its hidden states
    _, got = spec._mtp_rows(0, slot, nxt.cuda(), rt.hidden_rows, prefill=True)
    torch.cuda.synchronize()
    err = (got.float().cpu() - want).norm() / want.norm()
    assert err < 3e-2, err
    spec.free(slot)
