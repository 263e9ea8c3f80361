"""Prefix cache for hybrid (attention + recurrent) models: a request whose prompt starts with an already-seen prefix
re-uses that prefix's paged KV blocks and resumes the recurrent layers from a snapshot instead of recomputing them.

* Keys: blake2b digests of the token prefix at multiples of ``interval`` tokens (a multiple of the KV block size), so a
  lookup walks the prompt once and probes each boundary.
* Values: the KV block ids covering the prefix (shared by reference count with the sequences that use them) and an
  opaque snapshot of everything that is not positional: the Gated-DeltaNet states and the convolution tails.
* Eviction: least recently used, bounded by entry count and by snapshot bytes.

Reference behaviour: PrefixSnapshotCache (src/runtime/prefix_snapshot.py:45-271: LRU keyed by the blake2b of the token
prefix at 256-token blocks, restore on prefix hit) and the native engine's recurrent-state snapshots + prefix cache
(cpp_engine/include/qwen_engine.hpp:118-131, ``--qwen-snapshot-interval`` / ``--qwen-max-snapshots``).
"""
from __future__ import annotations

import hashlib
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Any, Callable, Sequence


@dataclass
class PrefixEntry:
    tokens: int
    blocks: list[int]
    snapshot: Any
    nbytes: int
    hits: int = 0


@dataclass
class PrefixCacheStats:
    lookups: int = 0
    hits: int = 0
    tokens_reused: int = 0
    inserts: int = 0
    evictions: int = 0


class PrefixCache:
    def __init__(self, interval: int = 256, max_entries: int = 16, max_bytes: int = 8 << 30,
                 release_blocks: Callable[[list[int]], None] | None = None):
        """``release_blocks`` is called with an evicted entry's block ids (the owner drops the cache's references)."""
        if interval <= 0:
            raise ValueError("interval must be positive")
        self.interval, self.max_entries, self.max_bytes = interval, max_entries, max_bytes
        self.release_blocks = release_blocks
        self._entries: "OrderedDict[bytes, PrefixEntry]" = OrderedDict()
        self.bytes = 0
        self.stats = PrefixCacheStats()

    # ---- keys
    def _digests(self, tokens: Sequence[int], upto: int) -> list[tuple[int, bytes]]:
        """(boundary, digest of tokens[:boundary]) for every multiple of ``interval`` up to ``upto``, incrementally."""
        h = hashlib.blake2b(digest_size=16)
        out = []
        for b in range(self.interval, upto + 1, self.interval):
            chunk = tokens[b - self.interval:b]
            h.update(b"".join(int(t).to_bytes(4, "little", signed=True) for t in chunk))
            out.append((b, h.copy().digest()))
        return out

    def boundaries(self, start: int, total: int) -> list[int]:
        """Snapshot points in (start, total): multiples of the interval strictly inside the prompt (the last token is
        always recomputed so that a hit still produces logits)."""
        first = (start // self.interval + 1) * self.interval
        return list(range(first, total, self.interval))

    # ---- lookup / insert
    def lookup(self, tokens: Sequence[int]) -> PrefixEntry | None:
        """Longest cached prefix of ``tokens`` that leaves at least one token to compute."""
        self.stats.lookups += 1
        best = None
        for b, d in self._digests(tokens, len(tokens) - 1):
            e = self._entries.get(d)
            if e is not None:
                best = (d, e)
        if best is None:
            return None
        d, e = best
        self._entries.move_to_end(d)
        e.hits += 1
        self.stats.hits += 1
        self.stats.tokens_reused += e.tokens
        return e

    def contains(self, tokens: Sequence[int], boundary: int) -> bool:
        ds = self._digests(tokens, boundary)
        return bool(ds) and ds[-1][0] == boundary and ds[-1][1] in self._entries

    def insert(self, tokens: Sequence[int], boundary: int, blocks: list[int], snapshot: Any, nbytes: int) -> bool:
        """Remember the state after ``tokens[:boundary]``.  Returns False (and keeps nothing) when the boundary is not a
        multiple of the interval, is already cached, or the snapshot alone exceeds the byte budget."""
        if boundary <= 0 or boundary % self.interval or boundary > len(tokens) or nbytes > self.max_bytes:
            return False
        d = self._digests(tokens, boundary)[-1][1]
        if d in self._entries:
            self._entries.move_to_end(d)
            return False
        self._entries[d] = PrefixEntry(boundary, list(blocks), snapshot, nbytes)
        self.bytes += nbytes
        self.stats.inserts += 1
        while len(self._entries) > self.max_entries or self.bytes > self.max_bytes:
            self._evict_oldest()
        return True

    def _evict_oldest(self) -> None:
        _, e = self._entries.popitem(last=False)
        self.bytes -= e.nbytes
        self.stats.evictions += 1
        if self.release_blocks is not None:
            self.release_blocks(e.blocks)

    def clear(self) -> None:
        while self._entries:
            self._evict_oldest()

    def __len__(self) -> int:
        return len(self._entries)
