"""CPU-rank stand-in for the peer-memory collectives: the same symmetric-buffer layout (per-rank flag words with
epochs, two parities of per-source data slots) and the same protocol (push my chunk into every peer's slot, publish
the epoch with a release, wait - bounded - for every peer's epoch, reduce in rank order) over POSIX shared memory,
with processes as ranks.  It exists so that the failure paths of the protocol can be exercised without a GPU: a peer
that is late, one that never arrives (``CollectiveTimeoutError``), a stale epoch left in a flag, out-of-order arrival.

The device implementation is csrc/comm/comm.cu (allreduce_oneshot_kernel); the reference's counterpart is its CUDA-IPC
one-shot all-reduce with a bounded spin and a status word (src/csrc/cuda_kernel_impl.cu:4788-4914)."""
from __future__ import annotations

import struct
import time
from multiprocessing import resource_tracker, shared_memory

import numpy as np

from .tp import CollectiveTimeoutError

MAX_RANKS = 8


class ShmPeerComm:
    """One instance per rank process.  ``name`` identifies the job; rank 0 creates the segments."""

    def __init__(self, name: str, rank: int, world: int, slot_elems: int = 1 << 16, budget_s: float = 2.0, create: bool | None = None):
        assert 1 <= world <= MAX_RANKS and 0 <= rank < world
        self.rank, self.world, self.slot_elems, self.budget_s = rank, world, slot_elems, budget_s
        self.flag_bytes = 2 * MAX_RANKS * 8                       # [parity][source] int64 epochs
        self.data_bytes = 2 * MAX_RANKS * slot_elems * 4          # [parity][source][slot] fp32
        size = 64 + self.flag_bytes + self.data_bytes
        create = rank == 0 if create is None else create
        self.bufs = []
        for r in range(world):
            seg = f"{name}_r{r}"
            if r == rank:
                if create or True:
                    try:
                        old = shared_memory.SharedMemory(name=seg)
                        old.close()
                        old.unlink()
                    except FileNotFoundError:
                        pass
                shm = shared_memory.SharedMemory(name=seg, create=True, size=size)
                shm.buf[:64 + self.flag_bytes] = bytes(64 + self.flag_bytes)
            else:
                shm = None
            self.bufs.append(shm)
        self.epoch = 0
        self._name = name

    def connect(self, timeout_s: float = 30.0) -> None:
        """Attach to the peers' segments (every rank creates its own first)."""
        t0 = time.monotonic()
        for r in range(self.world):
            while self.bufs[r] is None:
                try:
                    shm = shared_memory.SharedMemory(name=f"{self._name}_r{r}")
                    try:
                        resource_tracker.unregister(shm._name, "shared_memory")
                    except Exception:
                        pass
                    self.bufs[r] = shm
                except FileNotFoundError:
                    if time.monotonic() - t0 > timeout_s:
                        raise CollectiveTimeoutError(f"rank {r} never created its buffer")
                    time.sleep(0.005)

    # ---- addressing (mirrors flag_slot / data_slot of the device code)
    def _flag_off(self, parity: int, src: int) -> int:
        return 64 + (parity * MAX_RANKS + src) * 8

    def _data(self, r: int, parity: int, src: int) -> np.ndarray:
        off = 64 + self.flag_bytes + (parity * MAX_RANKS + src) * self.slot_elems * 4
        return np.frombuffer(self.bufs[r].buf, dtype=np.float32, count=self.slot_elems, offset=off)

    def all_reduce(self, x: np.ndarray, skip_push_to: set[int] = frozenset(), delay_s: float = 0.0) -> np.ndarray:
        """Sum of every rank's ``x`` (fp32 [n], n <= slot_elems), identical bits on every rank.
        ``skip_push_to`` / ``delay_s`` are fault-injection hooks for the tests: withhold this rank's flag from some
        peers, or arrive late."""
        n = x.size
        if n > self.slot_elems:
            raise ValueError("payload larger than a slot")
        self.epoch += 1
        epoch, parity = self.epoch, self.epoch & 1
        if delay_s:
            time.sleep(delay_s)
        for r in range(self.world):
            if r == self.rank:
                continue
            self._data(r, parity, self.rank)[:n] = x
        for r in range(self.world):                              # data first, then the flag (the release)
            if r == self.rank or r in skip_push_to:
                continue
            struct.pack_into("q", self.bufs[r].buf, self._flag_off(parity, self.rank), epoch)
        t0 = time.monotonic()
        for r in range(self.world):
            if r == self.rank:
                continue
            while struct.unpack_from("q", self.bufs[self.rank].buf, self._flag_off(parity, r))[0] < epoch:
                if time.monotonic() - t0 > self.budget_s:
                    raise CollectiveTimeoutError(f"rank {self.rank}: no data from rank {r} for epoch {epoch} within {self.budget_s} s")
                time.sleep(0)
        acc = np.zeros(n, dtype=np.float32)
        for r in range(self.world):                              # fixed order: bit-identical on every rank
            acc += x if r == self.rank else self._data(self.rank, parity, r)[:n]
        return acc

    def close(self) -> None:
        for r, shm in enumerate(self.bufs):
            if shm is None:
                continue
            self.bufs[r] = None
            try:
                shm.close()
                if r == self.rank:
                    shm.unlink()
            except Exception:
                pass
