"""Greedy speculative decoding on the host: draft a block, verify it in one target pass, keep the matching prefix plus
the target's own next token, roll the target back when the block broke.  The result is token-for-token the greedy
output of the target; only the number of target passes changes.

The target is any runtime with ``reset()``, ``forward(ids) -> logits [S, vocab]`` (appends ``ids`` to its context) and
``snapshot()`` / ``restore(snapshot)`` (recurrent layers cannot be truncated, so a broken block is undone by restoring
the state saved before the verify pass and replaying the accepted prefix).  A drafter has ``propose(context, k) ->
(tokens, confidence)``.  ``SpecGate`` (``spec_gate.py``) chooses how much of each block to verify.

Reference behaviour: the draft / verify / commit loop of src/models/deepseek_v4/dspark_loop.py:148-244 and the verify
transaction with state rollback of the native Qwen engine (cpp_engine/tests/test_batch_verify_transaction.cpp).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .spec_gate import SpecGate


class PromptLookupDrafter:
    """Model-free drafter: find the latest earlier occurrence of the context's last ``n`` tokens (longest ``n`` first)
    and propose what followed it.  Confidence is ``2 n - 2`` for every proposed position, i.e. longer matches land in
    higher gate buckets."""

    def __init__(self, max_ngram: int = 3, min_ngram: int = 1):
        assert max_ngram >= min_ngram >= 1
        self.max_ngram, self.min_ngram = max_ngram, min_ngram

    def propose(self, context: list[int], k: int) -> tuple[list[int], list[float]]:
        n_ctx = len(context)
        for n in range(min(self.max_ngram, n_ctx - 1), self.min_ngram - 1, -1):
            tail = context[n_ctx - n:]
            for s in range(n_ctx - n - 1, -1, -1):
                if context[s:s + n] == tail:
                    cont = context[s + n:s + n + k]
                    if cont:
                        return cont, [2.0 * n - 2.0] * len(cont)
        return [], []


@dataclass
class SpecStats:
    target_passes: int = 0
    replay_passes: int = 0
    rounds: int = 0
    drafted: int = 0
    accepted: int = 0
    plain_steps: int = 0
    gate: dict = field(default_factory=dict)

    @property
    def tokens_per_pass(self) -> float:
        return (self.accepted + self.rounds + self.plain_steps) / max(self.target_passes, 1)


@torch.no_grad()
def speculative_generate(target, drafter, prompt: torch.Tensor, max_new_tokens: int, block: int = 4,
                         gate: SpecGate | None = None, eos_token_id: int | None = None) -> tuple[list[int], SpecStats]:
    st = SpecStats()
    target.reset()
    logits = target.forward(prompt)
    st.target_passes += 1
    context = [int(t) for t in prompt.reshape(-1)]
    out: list[int] = []

    def commit(tok: int) -> bool:
        out.append(tok)
        context.append(tok)
        return len(out) >= max_new_tokens or (eos_token_id is not None and tok == eos_token_id)

    done = commit(int(logits[-1].argmax()))
    while not done:
        committed = out[-1]
        draft, conf, n = [], [], 0
        if gate is not None and not gate.should_draft(logits[-1].float().topk(2).values.tolist()):
            gate.note_skipped(by_margin=True)
        else:
            draft, conf = drafter.propose(context, min(block, max_new_tokens - len(out) - 1))
            n = len(draft)
            if gate is not None and n:
                pad = conf + [conf[-1]] * (gate.block - n)                # a short proposal is scored as if it continued
                n = min(gate.choose(pad), n)
                if n == 0:
                    gate.note_skipped()
        if n == 0:
            logits = target.forward(torch.tensor([committed]))
            st.target_passes += 1
            st.plain_steps += 1
            done = commit(int(logits[-1].argmax()))
            continue
        snap = target.snapshot()
        ver = target.forward(torch.tensor([committed] + draft[:n]))      # row i predicts the token after draft[i - 1]
        st.target_passes += 1
        pred = ver.argmax(-1).tolist()
        a = 0
        while a < n and pred[a] == draft[a]:
            a += 1
        st.rounds += 1
        st.drafted += n
        st.accepted += a
        if gate is not None:
            gate.observe(conf, a, n)
        for tok in draft[:a]:
            done = commit(tok)
            if done:
                break
        if not done:
            done = commit(pred[a])
        if done:
            break
        if a < n:                                                         # undo the rejected tail
            target.restore(snap)
            logits = target.forward(torch.tensor([committed] + draft[:a]))
            st.target_passes += 1
            st.replay_passes += 1
        else:
            logits = ver
    if gate is not None:
        st.gate = gate.stats()
    return out, st


# ---------------------------------------------------------------------------------------------- cache-free oracles
class WholeSequenceTarget:
    """Adapts an oracle with only ``forward(all_ids) -> logits [T, vocab]`` (no caches) to the target protocol by
    re-running the whole context; the state is just the token list, so snapshot / restore are exact and free.
    ``hidden`` / ``taps`` hold the oracle's ``last_hidden`` / ``last_taps`` of this target's latest pass when it has them
    (several targets may share one oracle)."""

    def __init__(self, oracle):
        self.oracle, self.ids, self.hidden, self.taps = oracle, [], None, None

    def reset(self) -> None:
        self.ids, self.hidden, self.taps = [], None, None

    def snapshot(self) -> list[int]:
        return list(self.ids)

    def restore(self, snap: list[int]) -> None:
        self.ids = list(snap)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        n = ids.numel()
        self.ids.extend(int(t) for t in ids.reshape(-1))
        logits = self.oracle.forward(torch.tensor(self.ids))
        self.hidden = getattr(self.oracle, "last_hidden", None)
        self.taps = getattr(self.oracle, "last_taps", None)          # tap-layer hidden states, when the oracle keeps them
        return logits[-n:]


class MtpDrafter:
    """Drafts with a multi-token-prediction head applied recursively: step 1 fuses the trunk's hidden states with the
    embeddings of the tokens that follow them (the last being the committed token), step j > 1 shifts the tokens by
    one, appends the previous draft and consumes the head's own hidden states.  Confidence is the margin between the
    two best draft logits.  ``target`` must be the ``WholeSequenceTarget`` of an oracle with ``mtp_forward``."""

    def __init__(self, target: WholeSequenceTarget):
        self.t = target

    def propose(self, context: list[int], k: int) -> tuple[list[int], list[float]]:
        hidden = self.t.hidden
        if k <= 0 or hidden is None or hidden.shape[0] != len(context) - 1:
            return [], []
        nxt = torch.tensor(context[1:])
        toks, conf = [], []
        for _ in range(k):
            logits, hidden = self.t.oracle.mtp_forward(nxt, hidden)
            top = logits[-1].float().topk(2).values
            toks.append(int(logits[-1].argmax()))
            conf.append(float(top[0] - top[1]))
            nxt = torch.cat([nxt[1:], torch.tensor([toks[-1]])])
        return toks, conf
