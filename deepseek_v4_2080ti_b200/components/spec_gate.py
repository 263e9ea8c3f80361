"""Adaptive draft length for speculative decoding.

A round drafts up to ``block`` tokens and the target model verifies a prefix of them in one forward pass whose cost
grows about linearly with the number verified.  A drafter that emits a confidence score per position lets the host
decide how many to verify: the gate keeps, per confidence bucket, a decayed count of (accepted, resolved) positions,
turns it into P(accept | confidence) with a pseudo-count prior, and picks

    n* = argmax_n  (1 + sum_{i<n} prod_{j<=i} p_j) / cost(n),     cost(0) = plain step, cost(n>0) = draft + verify(n)

the expected tokens per millisecond (the 1 is the token every verify yields anyway).  Positions after the first
mismatch are censored, not counted as misses.  Before drafting, the margin between the two best target logits can veto
the round when the target itself is unsure.

Reference behaviour: src/models/deepseek_v4/dspark_gate.py:94-255 (DSparkGate: match_prob, should_draft,
choose_draft_len, observe, stats).  Only the shape of the cost curve matters, so the constants are parameters.
"""
from __future__ import annotations

import bisect
import os
from dataclasses import dataclass, field
from typing import Iterable, Sequence


@dataclass
class SpecCost:
    """Milliseconds: one plain decode step, one draft, and verify(n) = base + slope * n."""
    plain_ms: float = 8.0
    draft_ms: float = 2.0
    verify_base_ms: float = 8.0
    verify_slope_ms: float = 0.3

    def round_ms(self, n: int) -> float:
        return self.plain_ms if n == 0 else self.draft_ms + self.verify_base_ms + self.verify_slope_ms * n


@dataclass
class SpecGate:
    block: int
    cost: SpecCost = field(default_factory=SpecCost)
    edges: Sequence[float] = (-0.5, 0.5, 1.5, 3.0, 6.0)      # bucket boundaries on the confidence score
    prior_n: float = 2.0                                     # optimistic prior: a fresh stream drafts the full block
    prior_p: float = 0.75
    decay: float = 0.9                                       # per-round forgetting, so a change of regime is tracked
    keep_full_margin: float = 1.15                           # a shorter draft must win by this factor
    min_draft: int = 0
    margin_threshold: float = 0.0                            # > 0: veto a round when top1 - top2 of the target is below it
    enabled: bool = True

    def __post_init__(self):
        if self.block <= 0:
            raise ValueError(f"block must be positive, got {self.block}")
        self._hit = [0.0] * (len(self.edges) + 1)
        self._seen = [0.0] * (len(self.edges) + 1)
        self.rounds = self.truncated = self.skipped = self.margin_skipped = 0

    @classmethod
    def from_env(cls, block: int, prefix: str = "POCKETLLM_SPEC_GATE") -> "SpecGate":
        """Off unless ``<prefix>=1``; ``<prefix>_PLAIN_MS``, ``_DRAFT_MS``, ``_VERIFY_BASE_MS``, ``_VERIFY_SLOPE_MS``,
        ``_MARGIN``, ``_MIN_DRAFT``, ``_DECAY`` and ``_MARGIN_THRESHOLD`` override the defaults."""
        f = lambda name, default: float(os.environ.get(f"{prefix}_{name}", default))
        base = SpecCost()
        cost = SpecCost(f("PLAIN_MS", base.plain_ms), f("DRAFT_MS", base.draft_ms), f("VERIFY_BASE_MS", base.verify_base_ms),
                        f("VERIFY_SLOPE_MS", base.verify_slope_ms))
        return cls(block, cost, keep_full_margin=f("MARGIN", 1.15), min_draft=int(f("MIN_DRAFT", 0)), decay=f("DECAY", 0.9),
                   margin_threshold=f("MARGIN_THRESHOLD", 0.0),
                   enabled=os.environ.get(prefix, "0").lower() in ("1", "true", "yes", "on"))

    # ---- estimate
    def bucket(self, conf: float) -> int:
        return bisect.bisect_right(list(self.edges), conf)

    def accept_prob(self, conf: float) -> float:
        b = self.bucket(conf)
        return (self._hit[b] + self.prior_n * self.prior_p) / (self._seen[b] + self.prior_n)

    # ---- decisions
    def should_draft(self, top2: Sequence[float]) -> bool:
        """``top2``: the two largest target logits of the committed position."""
        if not self.enabled or self.margin_threshold <= 0:
            return True
        return float(top2[0]) - float(top2[1]) >= self.margin_threshold

    def expected_rate(self, confidence: Sequence[float], n: int) -> float:
        """Expected tokens per millisecond of verifying the first ``n`` drafted tokens."""
        run, tokens = 1.0, 1.0
        for c in confidence[:n]:
            run *= self.accept_prob(float(c))
            tokens += run
        return tokens / self.cost.round_ms(n)

    def choose(self, confidence: Iterable[float]) -> int:
        """How many leading draft tokens to verify; 0 = take a plain step instead."""
        conf = [float(c) for c in confidence]
        if not self.enabled or len(conf) < self.block:
            return self.block
        rates = [self.expected_rate(conf, n) for n in range(self.block + 1)]
        best = max(range(self.block + 1), key=lambda n: (rates[n], n))
        if best != self.block and rates[best] < rates[self.block] * self.keep_full_margin:
            best = self.block
        if 0 < best < self.min_draft:
            best = min(self.min_draft, self.block)
        return best

    # ---- feedback
    def observe(self, confidence: Iterable[float], accepted: int, drafted: int) -> None:
        """A verified round: positions [0, accepted) matched, position ``accepted`` (if verified) did not, the rest
        is unknown."""
        if drafted <= 0:
            return
        conf = [float(c) for c in confidence]
        self.rounds += 1
        self.truncated += int(drafted < self.block)
        self._hit = [h * self.decay for h in self._hit]
        self._seen = [s * self.decay for s in self._seen]
        for i in range(min(accepted + 1, drafted, len(conf))):
            b = self.bucket(conf[i])
            self._hit[b] += 1.0 if i < accepted else 0.0
            self._seen[b] += 1.0

    def note_skipped(self, by_margin: bool = False) -> None:
        """A round that took a plain step: nothing is learned from it, so count it for the caller to notice a gate that
        never drafts."""
        self.rounds += 1
        self.skipped += 1
        self.margin_skipped += int(by_margin)

    def stats(self) -> dict:
        lo = [float("-inf")] + list(self.edges)
        hi = list(self.edges) + [float("inf")]
        return {"rounds": self.rounds, "truncated_rounds": self.truncated, "skipped_rounds": self.skipped,
                "margin_skipped_rounds": self.margin_skipped,
                "bucket_rates": {f"[{a:+.1f},{b:+.1f})": (round(h / s, 3) if s else None)
                                 for a, b, h, s in zip(lo, hi, self._hit, self._seen)}}
