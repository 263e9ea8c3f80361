"""Routed experts served by a separate host process: a POSIX shared-memory mailbox (request / response sequence
numbers, per-rank acknowledgements of output slots), a shared read-only arena holding one copy of the expert weights for
all ranks, and the server loop that answers requests with the C++ FP4 expert kernel.

On a B200 box every expert fits in HBM, so this path is the fallback for models larger than the GPUs (and the
counterpart of the reference's heterogeneous placement), not the default.  Waits poll with a timeout instead of
spinning forever: a dead peer raises ``TimeoutError``.

Reference behaviour: CPUMoESharedMemory (src/components/moe/ipc.py:14-130), SharedCPUMoEWeightArena
(src/components/moe/shared_weights.py:51-285: ready flags, 600 s timeout), the server process
(src/models/deepseek_v4/moe_server.py:36-104, 168+)."""
from __future__ import annotations

import struct
import time
from multiprocessing import resource_tracker, shared_memory

import torch

_HDR = "qqqq"                 # request_seq, response_seq, layer_id, stop
_HDR_BYTES = 64
_SLOTS = 4                    # response slots: a rank may still be reading seq while seq + 1 is produced
_MAX_RANKS = 16


def _attach(name: str, create: bool, size: int) -> shared_memory.SharedMemory:
    if create:
        try:
            stale = shared_memory.SharedMemory(name=name, create=False)
            stale.close()
            stale.unlink()
        except FileNotFoundError:
            pass
    shm = shared_memory.SharedMemory(name=name, create=create, size=size if create else 0)
    if not create:
        try:                   # the creator owns the segment; attaching processes must not unlink it at exit
            resource_tracker.unregister(shm._name, "shared_memory")
        except Exception:
            pass
    return shm


class MoEMailbox:
    """One outstanding request at a time: rows [T, dim] fp32 with their top-k expert ids and weights in, rows out."""

    def __init__(self, name: str, dim: int, topk: int, max_tokens: int = 1, create: bool = False):
        self.dim, self.topk, self.max_tokens = dim, topk, max_tokens
        self.in_bytes, self.ids_bytes, self.w_bytes = max_tokens * dim * 4, max_tokens * topk * 8, max_tokens * topk * 4
        self.out_bytes = max_tokens * dim * 4
        self.off_in = _HDR_BYTES
        self.off_ids = self.off_in + self.in_bytes
        self.off_w = self.off_ids + self.ids_bytes
        self.off_out = self.off_w + self.w_bytes
        self.off_ack = self.off_out + self.out_bytes * _SLOTS
        self.size = self.off_ack + _SLOTS * _MAX_RANKS * 8
        self.shm = _attach(name, create, self.size)
        self.buf = self.shm.buf
        if create:
            struct.pack_into(_HDR, self.buf, 0, 0, 0, -1, 0)
            struct.pack_into("q", self.buf, 32, 0)          # token count of the current request
            self.buf[self.off_ack:self.size] = bytes(self.size - self.off_ack)

    def close(self, unlink: bool = False) -> None:
        self.buf = None
        self.shm.close()
        if unlink:
            self.shm.unlink()

    def _t(self, dtype, count, offset, shape):
        return torch.frombuffer(self.buf, dtype=dtype, count=count, offset=offset).view(*shape)

    def header(self) -> tuple[int, int, int, int]:
        return struct.unpack_from(_HDR, self.buf, 0)

    # ---- client side
    def submit(self, layer: int, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor) -> int:
        t = x.shape[0]
        if t > self.max_tokens:
            raise ValueError(f"{t} rows exceed the mailbox capacity {self.max_tokens}")
        req, resp, _, _ = self.header()
        self._t(torch.float32, t * self.dim, self.off_in, (t, self.dim)).copy_(x.detach().float().cpu())
        self._t(torch.int64, t * self.topk, self.off_ids, (t, self.topk)).copy_(ids.detach().long().cpu())
        self._t(torch.float32, t * self.topk, self.off_w, (t, self.topk)).copy_(weights.detach().float().cpu())
        struct.pack_into("q", self.buf, 32, t)
        struct.pack_into("qq", self.buf, 16, layer, 0)
        struct.pack_into("q", self.buf, 0, req + 1)          # publish last
        return req + 1

    def wait_response(self, seq: int, timeout_s: float = 600.0) -> torch.Tensor:
        t0 = time.monotonic()
        while True:
            _, resp, _, stop = self.header()
            if stop:
                raise RuntimeError("expert server stopped")
            if resp >= seq:
                t = struct.unpack_from("q", self.buf, 32)[0]
                return self._t(torch.float32, t * self.dim, self.off_out + (seq % _SLOTS) * self.out_bytes, (t, self.dim))
            if time.monotonic() - t0 > timeout_s:
                raise TimeoutError(f"no response to request {seq} within {timeout_s} s")
            time.sleep(0)

    def ack(self, rank: int, seq: int) -> None:
        struct.pack_into("q", self.buf, self.off_ack + ((seq % _SLOTS) * _MAX_RANKS + rank) * 8, seq)

    # ---- server side
    def wait_request(self, last_seq: int, timeout_s: float | None = None) -> tuple[int, int] | None:
        """(seq, layer) of the next request, or None when told to stop."""
        t0 = time.monotonic()
        while True:
            req, _, layer, stop = self.header()
            if stop:
                return None
            if req > last_seq:
                return req, layer
            if timeout_s is not None and time.monotonic() - t0 > timeout_s:
                raise TimeoutError("no request")
            time.sleep(0)

    def request_tensors(self):
        t = struct.unpack_from("q", self.buf, 32)[0]
        return (self._t(torch.float32, t * self.dim, self.off_in, (t, self.dim)),
                self._t(torch.int64, t * self.topk, self.off_ids, (t, self.topk)),
                self._t(torch.float32, t * self.topk, self.off_w, (t, self.topk)))

    def wait_slot_free(self, seq: int, readers: list[int], timeout_s: float = 600.0) -> None:
        """Before overwriting the slot of ``seq``: every reader rank has acknowledged the response ``seq - SLOTS``."""
        old = seq - _SLOTS
        if old <= 0:
            return
        t0 = time.monotonic()
        while any(struct.unpack_from("q", self.buf, self.off_ack + ((old % _SLOTS) * _MAX_RANKS + r) * 8)[0] < old for r in readers):
            if time.monotonic() - t0 > timeout_s:
                raise TimeoutError(f"slot of response {old} was never acknowledged")
            time.sleep(0)

    def respond(self, seq: int, out: torch.Tensor) -> None:
        t = out.shape[0]
        self._t(torch.float32, t * self.dim, self.off_out + (seq % _SLOTS) * self.out_bytes, (t, self.dim)).copy_(out.float())
        struct.pack_into("q", self.buf, 8, seq)

    def stop(self) -> None:
        struct.pack_into("q", self.buf, 24, 1)


class SharedWeightArena:
    """One shared-memory copy of named tensors for all ranks of a host: the creator writes them and raises the ready
    flag; the others attach, wait for the flag (with a timeout) and get zero-copy views."""

    def __init__(self, name: str, layout: list[tuple[str, tuple[int, ...], torch.dtype]], create: bool = False):
        self.layout, off = {}, 64
        for n, shape, dt in layout:
            nb = torch.tensor([], dtype=dt).element_size()
            for s in shape:
                nb *= s
            self.layout[n] = (off, shape, dt)
            off += (nb + 63) // 64 * 64
        self.size = off
        self.shm = _attach(name, create, self.size)
        self.buf = self.shm.buf
        if create:
            struct.pack_into("q", self.buf, 0, 0)

    def view(self, name: str) -> torch.Tensor:
        off, shape, dt = self.layout[name]
        n = 1
        for s in shape:
            n *= s
        return torch.frombuffer(self.buf, dtype=dt, count=n, offset=off).view(*shape)

    def publish(self, tensors: dict[str, torch.Tensor]) -> None:
        for n, t in tensors.items():
            self.view(n).copy_(t)
        struct.pack_into("q", self.buf, 0, 1)

    def wait_ready(self, timeout_s: float = 600.0) -> None:
        t0 = time.monotonic()
        while struct.unpack_from("q", self.buf, 0)[0] != 1:
            if time.monotonic() - t0 > timeout_s:
                raise TimeoutError("shared expert weights were not published in time")
            time.sleep(0.001)

    def close(self, unlink: bool = False) -> None:
        self.buf = None
        self.shm.close()
        if unlink:
            self.shm.unlink()


def serve_experts(mailbox: MoEMailbox, expert_fn, readers: list[int] | None = None, max_requests: int | None = None) -> int:
    """Server loop: ``expert_fn(layer, x, ids, weights) -> [T, dim]`` for every request until stopped.
    Returns the number of requests served."""
    last, n = 0, 0
    while max_requests is None or n < max_requests:
        nxt = mailbox.wait_request(last)
        if nxt is None:
            break
        seq, layer = nxt
        x, ids, w = mailbox.request_tensors()
        out = expert_fn(layer, x.clone(), ids.clone(), w.clone())
        if readers:
            mailbox.wait_slot_free(seq, readers)
        mailbox.respond(seq, out)
        last, n = seq, n + 1
    return n
