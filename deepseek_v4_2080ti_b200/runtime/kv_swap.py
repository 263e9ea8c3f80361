"""Host-resident KV chunks with a device-side working set (the storage half of FlashMemory).

The KV rows of the far context are kept chunk by chunk (``chunk_tokens`` rows of ``row_bytes``) in pinned host memory;
the device holds ``device_chunks`` slots.  ``store`` writes a finished chunk to the host (device-to-host copy on a side
stream), ``ensure`` makes the chunks the retriever kept resident - hits cost nothing, misses evict the least recently
used slots and are fetched with one host-to-device copy per chunk on the side stream - and returns the slot of each
chunk; the compute stream waits on one event.  With 180 GB on the device the working set can be large, so the common
case is a pure hit.

Reference behaviour: the KV swap of the FlashMemory plugin (cpp_engine/engine/deepseek_v4_engine.cpp:5362-5640: host
pool, top-k driven fetch, window + retrieved layout); decode throughput with and without the swap is within 2 % there
(docs/FLASHMEMORY_1M_CONTEXT.md:203-204).
"""
from __future__ import annotations

from collections import OrderedDict

import torch


class KvSwapManager:
    def __init__(self, host_chunks: int, device_chunks: int, chunk_tokens: int, row_bytes: int, device="cuda"):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.chunk_tokens, self.row_bytes = int(chunk_tokens), int(row_bytes)
        self.host = torch.empty(host_chunks, chunk_tokens, row_bytes, dtype=torch.uint8, pin_memory=self.cuda)
        self.dev = torch.zeros(device_chunks, chunk_tokens, row_bytes, dtype=torch.uint8, device=self.device)
        self.stored = [False] * host_chunks
        self.slot_of: OrderedDict[int, int] = OrderedDict()          # chunk -> slot, least recently used first
        self.free_slots = list(range(device_chunks - 1, -1, -1))
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.hits = self.misses = self.evictions = 0
        self.h2d_bytes = self.d2h_bytes = 0

    # ---- host side of the pool
    def store(self, chunk: int, rows: torch.Tensor, keep_resident: bool = False) -> None:
        """``rows``: uint8 view [chunk_tokens, row_bytes] of the chunk's KV rows on the device.  The copy to the host
        is ordered after the work already queued on the current stream."""
        assert rows.dtype == torch.uint8 and tuple(rows.shape) == (self.chunk_tokens, self.row_bytes)
        if self.cuda:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.stream):
                self.host[chunk].copy_(rows, non_blocking=True)
            rows.record_stream(self.stream)
        else:
            self.host[chunk].copy_(rows)
        self.stored[chunk] = True
        self.d2h_bytes += rows.numel()
        if keep_resident:
            slot = self._take_slot(chunk, protect=())
            self.dev[slot].copy_(rows)

    def _take_slot(self, chunk: int, protect) -> int:
        if chunk in self.slot_of:
            self.slot_of.move_to_end(chunk)
            return self.slot_of[chunk]
        if self.free_slots:
            slot = self.free_slots.pop()
        else:
            victim = next((c for c in self.slot_of if c not in protect), None)
            if victim is None:
                raise RuntimeError("device working set is smaller than the number of chunks requested at once")
            slot = self.slot_of.pop(victim)
            self.evictions += 1
        self.slot_of[chunk] = slot
        return slot

    # ---- device side
    def ensure(self, chunk_ids) -> torch.Tensor:
        """Make every chunk of ``chunk_ids`` (ints, -1 = none) resident; returns int32 [len] device slots (-1 for
        none).  The current stream waits for the fetches."""
        ids = [int(c) for c in (chunk_ids.tolist() if isinstance(chunk_ids, torch.Tensor) else chunk_ids)]
        want = {c for c in ids if c >= 0}
        if len(want) > self.dev.shape[0]:
            raise RuntimeError("device working set is smaller than the number of chunks requested at once")
        if self.cuda:
            # a slot about to be overwritten may still be read by attention kernels already queued
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
        slots = []
        fetched = False
        for c in ids:
            if c < 0:
                slots.append(-1)
                continue
            if c in self.slot_of:
                self.hits += 1
                slots.append(self._take_slot(c, want))
                continue
            if not self.stored[c]:
                raise KeyError(f"chunk {c} was never stored")
            self.misses += 1
            slot = self._take_slot(c, want)
            if self.cuda:
                with torch.cuda.stream(self.stream):
                    self.dev[slot].copy_(self.host[c], non_blocking=True)
            else:
                self.dev[slot].copy_(self.host[c])
            self.h2d_bytes += self.host[c].numel()
            fetched = True
            slots.append(slot)
        if self.cuda and fetched:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
        return torch.tensor(slots, dtype=torch.int32, device=self.device)

    def rows(self, slots: torch.Tensor) -> torch.Tensor:
        """Row indices into ``dev.view(-1, row_bytes)`` of the given slots' tokens, int32 [len * chunk_tokens] (-1 kept)."""
        base = slots.to(torch.int64)[:, None] * self.chunk_tokens + torch.arange(self.chunk_tokens, device=slots.device)
        return torch.where(slots[:, None] < 0, torch.full_like(base, -1), base).reshape(-1).to(torch.int32)

    def synchronize(self) -> None:
        if self.cuda:
            self.stream.synchronize()

    def stats(self) -> dict:
        return {"hits": self.hits, "misses": self.misses, "evictions": self.evictions, "resident": len(self.slot_of),
                "h2d_bytes": self.h2d_bytes, "d2h_bytes": self.d2h_bytes}
