"""Hot-expert cache: routed-expert weights live in host memory and only the experts a step needs occupy device slots.

For models whose experts do not fit beside the KV cache (or when several models share a GPU), each MoE layer keeps
its experts as equal-sized byte slabs in (pinned) host memory and owns ``capacity`` device slots.  ``fetch(ids)``
returns the slot of every requested expert, copying the missing ones in on a side stream; least-recently-used experts
are evicted, never one that the same call asked for.  ``prefetch(ids)`` starts the copies without waiting, so the
router's result for layer L + 1 can be staged while layer L computes; the grouped GEMM reads ``slots`` directly, slot
indices standing in for expert ids.

The logic is device-agnostic (CPU tensors work, which is what the tests use); on CUDA the host store is pinned and
copies run on their own stream, ordered against the compute stream with events.

Reference behaviour: GPUPrefillMoEBackend and its _HotExpertCache (src/components/moe/gpu_prefill_backend.py:41-104,
105-901: pinned host slabs, H2D streaming of the needed experts, hot set kept resident).
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass
from typing import Iterable

import torch


@dataclass
class ExpertCacheStats:
    hits: int = 0
    misses: int = 0
    evictions: int = 0
    bytes_copied: int = 0

    @property
    def hit_rate(self) -> float:
        return self.hits / max(self.hits + self.misses, 1)


class HotExpertCache:
    def __init__(self, host_slabs: torch.Tensor, capacity: int, device: torch.device | str = "cpu"):
        """host_slabs uint8 [n_experts, slab_bytes]: one expert's matrices, packed however the GEMM wants them."""
        assert host_slabs.dim() == 2 and host_slabs.dtype == torch.uint8 and capacity >= 1
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.n_experts, self.slab_bytes = host_slabs.shape
        self.capacity = min(int(capacity), self.n_experts)
        self.host = host_slabs.contiguous()
        if self.cuda and not self.host.is_pinned():
            self.host = self.host.pin_memory()
        self.slots = torch.empty(self.capacity, self.slab_bytes, dtype=torch.uint8, device=self.device)
        self._slot_of: "OrderedDict[int, int]" = OrderedDict()        # expert -> slot, least recently used first
        self._free = list(range(self.capacity - 1, -1, -1))
        self._stream = torch.cuda.Stream(self.device) if self.cuda else None
        self._ready: dict[int, "torch.cuda.Event"] = {}               # slot -> copy finished
        self.stats = ExpertCacheStats()

    # ---- residency
    def resident(self) -> list[int]:
        return list(self._slot_of)

    def _claim(self, expert: int, keep: set[int]) -> int:
        if self._free:
            return self._free.pop()
        for victim in self._slot_of:                                   # oldest first
            if victim not in keep:
                self.stats.evictions += 1
                return self._slot_of.pop(victim)
        raise RuntimeError(f"{len(keep)} experts requested at once, the cache holds {self.capacity}")

    def _load(self, expert: int, slot: int) -> None:
        self.stats.bytes_copied += self.slab_bytes
        if not self.cuda:
            self.slots[slot].copy_(self.host[expert])
            return
        # the slot may still be read by kernels already queued on the compute stream
        self._stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self._stream):
            self.slots[slot].copy_(self.host[expert], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self._stream)
        self._ready[slot] = ev

    def prefetch(self, experts: Iterable[int]) -> list[int]:
        """Make ``experts`` resident (copies may still be in flight); returns their slots in request order."""
        want = [int(e) for e in experts]
        keep = set(want)
        if len(keep) > self.capacity:
            raise RuntimeError(f"{len(keep)} experts requested at once, the cache holds {self.capacity}")
        out = []
        for e in want:
            if not 0 <= e < self.n_experts:
                raise IndexError(f"expert {e} out of range [0, {self.n_experts})")
            slot = self._slot_of.get(e)
            if slot is None:
                self.stats.misses += 1
                slot = self._claim(e, keep)
                self._load(e, slot)
                self._slot_of[e] = slot
            else:
                self.stats.hits += 1
                self._slot_of.move_to_end(e)
            out.append(slot)
        return out

    def fetch(self, experts: Iterable[int]) -> torch.Tensor:
        """Slots of ``experts`` as an int32 tensor on the device, with every copy ordered before what the current
        stream does next."""
        slots = self.prefetch(experts)
        if self.cuda:
            cur = torch.cuda.current_stream(self.device)
            for s in set(slots):
                ev = self._ready.pop(s, None)
                if ev is not None:
                    cur.wait_event(ev)
        return torch.tensor(slots, dtype=torch.int32, device=self.device)

    def slab(self, expert: int) -> torch.Tensor:
        """Device bytes of a resident expert (after ``fetch``)."""
        return self.slots[self._slot_of[int(expert)]]

    def remap(self, expert_ids: torch.Tensor) -> torch.Tensor:
        """Routing indices (any shape) -> slot indices; every id must be resident."""
        table = torch.full((self.n_experts,), -1, dtype=torch.int32)
        for e, s in self._slot_of.items():
            table[e] = s
        out = table.to(expert_ids.device)[expert_ids.long()]
        if bool((out < 0).any()):
            raise RuntimeError("remap of an expert that is not resident")
        return out


def pack_slabs(expert_tensors: list[list[torch.Tensor]]) -> tuple[torch.Tensor, list[tuple[int, tuple, torch.dtype]]]:
    """[[w1, w3, w2] per expert] -> (uint8 [E, bytes], layout) with ``layout`` = (offset, shape, dtype) per matrix, the
    same for every expert; ``view_slab`` undoes it on a device slab."""
    layout, off = [], 0
    for t in expert_tensors[0]:
        layout.append((off, tuple(t.shape), t.dtype))
        off += (t.numel() * t.element_size() + 15) // 16 * 16                 # keep every matrix 16-byte aligned
    slabs = torch.zeros(len(expert_tensors), off, dtype=torch.uint8)
    for e, ts in enumerate(expert_tensors):
        for (o, shape, dt), t in zip(layout, ts):
            assert tuple(t.shape) == shape and t.dtype == dt
            raw = t.contiguous().view(torch.uint8).reshape(-1)
            slabs[e, o:o + raw.numel()] = raw
    return slabs, layout


def view_slab(slab: torch.Tensor, layout: list[tuple[int, tuple, torch.dtype]]) -> list[torch.Tensor]:
    out = []
    for o, shape, dt in layout:
        n = int(torch.tensor(shape).prod()) * torch.empty(0, dtype=dt).element_size()
        out.append(slab[o:o + n].view(dt).view(shape))
    return out
