"""DSpark-style block drafter over the V4 CPU runtime: ring bookkeeping, bigram chaining, confidence read-out, and the
draft / verify / commit loop against plain greedy decoding."""
import torch

from deepseek_v4_2080ti_b200.components.spec_gate import SpecCost, SpecGate
from deepseek_v4_2080ti_b200.models import v4_block_ref as v4
from deepseek_v4_2080ti_b200.models import v4_dspark_ref as ds


def _setup(rank=8, block=4, seed=0):
    cfg = v4.V4Config(mtp=False)
    tgt = v4.V4BlockRef(cfg, v4.synth_weights(cfg, seed))
    dw = ds.synth_dspark_weights(cfg, n_stages=3, n_target=2, markov_rank=rank, seed=seed)
    return cfg, tgt, ds.DSparkRef(tgt, dw, target_layer_ids=(1, 2), block=block, noise_token_id=1), dw


def _ids(cfg, n, seed=1):
    return torch.randint(2, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(seed))


def test_ring_holds_the_last_window_of_target_hidden_states():
    cfg, tgt, d, _ = _setup()
    ids = _ids(cfg, 21)
    tgt.forward(ids)
    h = d.target_hidden()
    assert h.shape == (21, 2 * cfg.dim) and len(d.stages) == 3
    d.write_kv(h, 0)
    ring = d.stages[0].kv[:cfg.window].clone()
    d.reset()
    for p in range(21):                                     # position by position gives the same ring
        d.write_kv(h[p:p + 1], p)
    assert torch.allclose(d.stages[0].kv[:cfg.window], ring, atol=1e-6)
    d.reset(); d.write_kv(h[-cfg.window:], 21 - cfg.window)
    assert torch.allclose(d.stages[0].kv[:cfg.window], ring, atol=1e-6)


def test_draft_block_chains_through_the_bigram_bias_and_scores_confidence():
    cfg, tgt, d, dw = _setup()
    ids = _ids(cfg, 12)
    tgt.forward(ids); h = d.target_hidden(); d.write_kv(h, 0)
    snap = [s.kv.clone() for s in d.stages]
    toks, logits, conf = d.draft(h[-1:], 5, 12)
    assert len(toks) == 4 and logits.shape == (4, cfg.vocab_size) and conf.shape == (4,)
    assert toks == [int(logits[i].argmax()) for i in range(4)]
    # without the bias every position is independent of the chosen tokens; with it position i moves with token i - 1
    for s, k in zip(d.stages, snap):
        s.kv.copy_(k)
    d.w["dspark.markov_w2"] = torch.zeros_like(d.w["dspark.markov_w2"])
    _, base, conf0 = d.draft(h[-1:], 5, 12)
    e = [d.w["dspark.markov_w1"][t] for t in [5] + toks[:-1]]
    for i in range(4):
        assert torch.allclose(logits[i] - base[i], dw["dspark.markov_w2"].float() @ e[i], atol=1e-5)
    # the confidence is linear in [hidden, bigram embedding]: same hidden, different embeddings
    dconf = conf - conf0
    w_e = d.w["dspark.confidence"][0, cfg.dim:]
    toks0 = [int(base[i].argmax()) for i in range(4)]
    e0 = [d.w["dspark.markov_w1"][t] for t in [5] + toks0[:-1]]
    assert torch.allclose(dconf, torch.stack([(a - b) @ w_e for a, b in zip(e, e0)]), atol=1e-5)
    # no causal mask inside the block: changing the noise token changes position 0 too
    for s, k in zip(d.stages, snap):
        s.kv.copy_(k)
    d.noise = 2
    _, other, _ = d.draft(h[-1:], 5, 12)
    assert (other[0] - base[0]).abs().max() > 1e-6


def test_loop_output_is_the_greedy_continuation_whatever_the_drafts():
    cfg, tgt, d, _ = _setup()
    prompt = _ids(cfg, 14, seed=4)
    greedy = tgt.generate(prompt, 12)
    loop = ds.DSparkLoop(d)
    assert loop.generate(prompt, 12) == greedy
    assert loop.drafted == 4 * loop.rounds and 0 <= loop.accepted <= loop.drafted
    gated = ds.DSparkLoop(d, SpecGate(4, SpecCost(8, 1, 8, 0.3)))
    assert gated.generate(prompt, 12) == greedy and gated.gate.rounds == gated.rounds


def test_a_drafter_that_knows_the_bigrams_is_accepted_and_saves_rounds():
    cfg, tgt, d, _ = _setup(rank=v4.V4Config().vocab_size)
    prompt = _ids(cfg, 14, seed=4)
    greedy = tgt.generate(prompt, 16)
    chain = [int(x) for x in greedy]
    succ = {}
    for a, b in zip(chain[:-1], chain[1:]):
        succ.setdefault(a, b)
    consistent = sum(succ[a] == b for a, b in zip(chain[:-1], chain[1:]))
    d.w["dspark.markov_w1"] = torch.eye(cfg.vocab_size)
    w2 = torch.zeros(cfg.vocab_size, cfg.vocab_size)
    for a, b in succ.items():
        w2[b, a] = 1e3                                      # the bias names the successor outright
    d.w["dspark.markov_w2"] = w2
    loop = ds.DSparkLoop(d)
    assert loop.generate(prompt, 16) == greedy
    assert loop.accepted >= consistent // 2 and loop.rounds < 16 and loop.target_steps >= 16
