"""Tensor-parallel communicator.

``TPComm`` is the NCCL baseline (what the reference does with ``all_reduce_half`` after every
row-parallel projection, cpp_engine/engine/qwen_engine.cpp:2010-2037, and the packed arg-max merge,
cpp_engine/backends/cuda/collective/tp_comm.cpp:345-364).  The fused paths replace ``all_reduce``
with in-kernel peer-memory reductions; they plug in through the same interface.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def init_distributed(backend: str | None = None) -> tuple[int, int, int]:
    """Initialise torch.distributed from the torchrun environment. Returns (rank, world, local_rank)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local)
            dist.init_process_group(backend, rank=rank, world_size=world, device_id=torch.device("cuda", local))
        else:
            dist.init_process_group(backend, rank=rank, world_size=world)
    return rank, world, local


class TPComm:
    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.bytes_reduced = 0

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
            self.bytes_reduced += t.numel() * t.element_size()
        return t

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        """[world, *t.shape]: every rank's tensor, in rank order."""
        if self.world == 1:
            return t.unsqueeze(0)
        out = torch.empty(self.world, *t.shape, dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
        return out

    def moe_combine(self, y: torch.Tensor, route_row: torch.Tensor, wts: torch.Tensor, base: torch.Tensor | None,
                    residual: torch.Tensor | None, t: int, k: int, h: int, mode: int = 0) -> torch.Tensor:
        """Library baseline of the expert-parallel combine: local weighted combine, NCCL all-reduce, residual add."""
        out = torch.empty(t, h, dtype=torch.bfloat16, device=y.device)
        rc = _lib.lib().b200_moe_combine(_lib.ptr(y), _lib.ptr(route_row), _lib.ptr(wts), _lib.ptr(base), _lib.ptr(out),
                                         t, k, h, _lib.stream())
        _lib.check(rc, "moe_combine")
        out = self.all_reduce(out)
        return out if residual is None else out.add_(residual)

    def argmax_merge(self, idx: torch.Tensor, val: torch.Tensor) -> torch.Tensor:
        """Global arg-max from per-rank (index, value) winners over vocab shards; ties go to the lower id."""
        if self.world == 1:
            return idx
        packed = torch.stack([val.float(), idx.float()], -1).contiguous()       # ids < 2^24 are exact in fp32
        gathered = torch.empty(self.world, *packed.shape, dtype=packed.dtype, device=packed.device)
        dist.all_gather_into_tensor(gathered, packed, group=self.group)
        vals, ids = gathered[..., 0], gathered[..., 1]
        best = vals.max(0, keepdim=True).values
        cand = torch.where(vals == best, ids, torch.full_like(ids, float("inf")))
        return cand.min(0).values.to(torch.int32)

    def barrier(self) -> None:
        if self.world > 1:
            dist.barrier(group=self.group)


# ----------------------------------------------------------------------------- peer-memory communicator
import ctypes  # noqa: E402

from ..ops import _lib  # noqa: E402

MAX_RANKS = 8


class _CommStruct(ctypes.Structure):
    """Mirror of ``B200Comm`` (csrc/comm/comm.h)."""
    _fields_ = [("rank", ctypes.c_int), ("world", ctypes.c_int), ("slot_elems", ctypes.c_ulonglong),
                ("flags", ctypes.c_void_p * MAX_RANKS), ("ctrl", ctypes.c_void_p),
                ("data", ctypes.c_void_p * MAX_RANKS), ("flags2", ctypes.c_void_p * MAX_RANKS),
                ("result", ctypes.c_void_p * MAX_RANKS)]


class CollectiveTimeoutError(RuntimeError):
    """A bounded device-side wait on a peer's flag expired (the peer is late, gone, or out of step)."""


class PeerComm(TPComm):
    """Tensor-parallel communicator over NVLink peer memory.

    Every rank allocates one symmetric buffer (flags | control words | data slots), exports it with CUDA IPC
    and maps every peer's buffer; collectives are then done by this package's kernels with plain peer stores
    and loads (no NCCL on the hot path):

    * ``all_reduce``           one-shot all-reduce for payloads up to ``slot_elems`` bf16 values
    * ``argmax_merge``         (value, index) winners of the vocabulary shards
    * ``linear_allreduce``     row-parallel GEMM whose epilogue pushes each finished tile to the peers and
                               sums theirs (csrc/kernels/gemm_wdec.cu, ``ar_mode``)

    Larger payloads and anything else fall back to the NCCL group.  Device waits are bounded
    (``budget_ms``); on expiry the kernels set the status word and ``check()`` raises
    ``CollectiveTimeoutError``.  The reference's counterpart is its CUDA-IPC one-shot all-reduce with NCCL
    fallback, fixed at four ranks (src/models/deepseek_v4/runtime.py:206-268, 4211-4217).
    """

    def __init__(self, group=None, slot_elems: int = 1 << 20, budget_ms: float = 2000.0):
        super().__init__(group)
        assert self.world <= MAX_RANKS
        self.slot_elems = int(slot_elems)
        self.budget_ns = int(budget_ms * 1e6)
        self.device = torch.device("cuda", torch.cuda.current_device())
        L = _lib.lib()
        base = self._alloc(self.slot_elems)
        self._base = base
        self._band = band = self._guard()      # the same on every rank: they share the environment
        handle = ctypes.create_string_buffer(64)
        rc = L.b200_comm_ipc_handle(base, handle)
        if rc != 0:
            raise RuntimeError(f"cudaIpcGetMemHandle failed: {rc}")
        handles: list = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=self.group)
        self._peers: list[ctypes.c_void_p] = []
        bases = (ctypes.c_void_p * MAX_RANKS)()
        for r in range(self.world):
            if r == self.rank:
                bases[r] = base.value + band
                continue
            p = ctypes.c_void_p()
            rc = L.b200_comm_ipc_open(ctypes.c_char_p(handles[r]), ctypes.byref(p))
            if rc != 0:
                raise RuntimeError(f"cudaIpcOpenMemHandle(rank {r}) failed: {rc}")
            self._peers.append(p)
            bases[r] = p.value + band
        self._bind(bases)
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    GUARD_BYTES = 65536      # guard band on each side of a symmetric buffer when B200_CANARY=1

    @classmethod
    def _guard(cls) -> int:
        from ..utils import canary
        return cls.GUARD_BYTES if canary.is_enabled() else 0

    @classmethod
    def _alloc(cls, slot_elems: int) -> ctypes.c_void_p:
        """Allocate one symmetric buffer.  With guards on, the allocation is ``band | buffer | band``; the returned
        pointer is that of the allocation (what the IPC handle names) and every user adds ``_guard()`` to reach the
        buffer."""
        L = _lib.lib()
        L.b200_comm_buffer_bytes.restype = ctypes.c_ulonglong
        nbytes = L.b200_comm_buffer_bytes(ctypes.c_ulonglong(slot_elems))
        band = cls._guard()
        base = ctypes.c_void_p()
        rc = L.b200_comm_alloc(ctypes.c_ulonglong(nbytes + 2 * band), ctypes.byref(base))
        if rc != 0:
            raise RuntimeError(f"symmetric buffer allocation failed: CUDA error {rc}")
        if band:
            for off in (0, band + nbytes):
                cls._bytes_view(base.value + off, band).fill_(0xA5)
        return base

    @staticmethod
    def _bytes_view(ptr: int, n: int) -> torch.Tensor:
        class _Mem:
            __cuda_array_interface__ = {"shape": (n,), "typestr": "|u1", "data": (ptr, False), "version": 2}

        return torch.as_tensor(_Mem(), device=torch.device("cuda", torch.cuda.current_device()))

    def verify_guards(self) -> list[str]:
        """Bytes next to this rank's symmetric buffer that no longer hold the guard pattern (empty without guards)."""
        band = getattr(self, "_band", 0)
        if not band or self._base is None:
            return []
        L = _lib.lib()
        nbytes = L.b200_comm_buffer_bytes(ctypes.c_ulonglong(self.slot_elems))
        out = []
        for side, off in (("before", 0), ("after", band + nbytes)):
            b = self._bytes_view(self._base.value + off, band)
            bad = (b != 0xA5).nonzero()
            if bad.numel():
                out.append(f"symmetric buffer of rank {self.rank}: {bad.numel()} byte(s) {side} it overwritten, first at +{int(bad[0])}")
                b.fill_(0xA5)
        return out

    def _bind(self, bases) -> None:
        self.c = _CommStruct()
        rc = _lib.lib().b200_comm_init(ctypes.byref(self.c), self.rank, self.world, bases,
                                       ctypes.c_ulonglong(self.slot_elems))
        if rc != 0:
            raise RuntimeError(f"comm init failed: {rc}")
        self.fused_calls = 0
        self.standalone_calls = 0
        self._result_index = 0
        self._rs_bn = 0
        self.sp_enabled = os.environ.get("B200_SP", "1") != "0"
        self.degraded = False       # after recover(): every collective goes through the process group (NCCL)
        self.recoveries = 0
        # all-gather push on a second stream, overlapping the GEMM that consumes the gathered rows (B200_SP_OVERLAP=0:
        # the gather kernel pushes the rows itself, on the compute stream)
        self.overlap_gather = os.environ.get("B200_SP_OVERLAP", "1") != "0"
        self._side_stream = None
        self._push_done = None
        self._epoch_word = 0

    @classmethod
    def local_group(cls, world: int, slot_elems: int, budget_ms: float = 50.0) -> list["PeerComm"]:
        """``world`` communicators over ``world`` symmetric buffers of ONE device, in one process: the ranks of a
        collective are then stepped one after another on one stream (phase by phase, so that every wait finds its
        flags already raised by kernels that have completed).  For single-GPU numerics tests of the multi-rank
        kernels and for the timeout path; the collectives that fall back to the process group are not available."""
        bases = (ctypes.c_void_p * MAX_RANKS)()
        raw = [cls._alloc(int(slot_elems)) for _ in range(world)]
        band = cls._guard()
        for r in range(world):
            bases[r] = raw[r].value + band
        out = []
        for r in range(world):
            c = cls.__new__(cls)
            c.group, c.world, c.rank, c.bytes_reduced = None, world, r, 0
            c.slot_elems, c.budget_ns = int(slot_elems), int(budget_ms * 1e6)
            c.device = torch.device("cuda", torch.cuda.current_device())
            c._base, c._peers, c._band = raw[r], [], band
            c._bind(bases)
            c.overlap_gather = False      # one device: a kernel must never wait for a kernel of another stream
            out.append(c)
        torch.cuda.synchronize()
        return out

    def _cref(self):
        return ctypes.byref(self.c)

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return t
        if self.degraded or t.dtype != torch.bfloat16 or not t.is_contiguous() or t.numel() > self.slot_elems:
            return super().all_reduce(t)
        rc = _lib.lib().b200_allreduce_oneshot(self._cref(), _lib.ptr(t), ctypes.c_longlong(t.numel()),
                                               _lib.ptr(_lib.status_word(t.device)), ctypes.c_ulonglong(self.budget_ns),
                                               _lib.stream())
        _lib.check(rc, "allreduce_oneshot")
        self.standalone_calls += 1        # a peer-memory collective, but not fused into a compute kernel
        self.bytes_reduced += t.numel() * 2
        return t

    def argmax_merge(self, idx: torch.Tensor, val: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return idx
        rows = idx.numel()
        if self.degraded or rows * 4 > self.slot_elems:
            return super().argmax_merge(idx, val)
        out = torch.empty(rows, dtype=torch.int32, device=idx.device)
        rc = _lib.lib().b200_argmax_merge(self._cref(), _lib.ptr(val.float().contiguous()),
                                          _lib.ptr(idx.to(torch.int32).contiguous()), rows, _lib.ptr(out),
                                          _lib.ptr(_lib.status_word(idx.device)), ctypes.c_ulonglong(self.budget_ns),
                                          _lib.stream())
        _lib.check(rc, "argmax_merge")
        return out

    def moe_combine(self, y: torch.Tensor, route_row: torch.Tensor, wts: torch.Tensor, base: torch.Tensor | None,
                    residual: torch.Tensor | None, t: int, k: int, h: int, mode: int = 0) -> torch.Tensor:
        """Expert-parallel combine fused with its collective: ``residual + sum_ranks(base_r + sum_k w * y_r[row])``.
        mode 0 picks one-shot or two-shot by payload size (csrc/comm/moe_comm.cu)."""
        if self.degraded:
            return super().moe_combine(y, route_row, wts, base, residual, t, k, h, mode)
        out = torch.empty(t, h, dtype=torch.bfloat16, device=y.device)
        rc = _lib.lib().b200_moe_combine_allreduce(self._cref(), _lib.ptr(y), _lib.ptr(route_row), _lib.ptr(wts),
                                                   _lib.ptr(base), _lib.ptr(residual), _lib.ptr(out), t, k, h, mode,
                                                   _lib.ptr(_lib.status_word(y.device)),
                                                   ctypes.c_ulonglong(self.budget_ns), _lib.stream())
        _lib.check(rc, "moe_combine_allreduce")
        self.fused_calls += 1
        self.bytes_reduced += t * h * 2
        return out

    def _result_view(self, index: int, t: int, n: int) -> torch.Tensor:
        """bf16 [t, n] view of this rank's result buffer ``index`` inside the symmetric allocation."""
        ptr = int(self.c.result[self.rank]) + index * self.slot_elems * 2

        class _Mem:
            __cuda_array_interface__ = {"shape": (t * n,), "typestr": "<u2", "data": (ptr, False), "version": 2}

        return torch.as_tensor(_Mem(), device=self.device).view(torch.bfloat16).view(t, n)

    def linear_allreduce(self, x: torch.Tensor, w, residual: torch.Tensor | None = None,
                         two_shot: bool | None = None) -> torch.Tensor:
        """``sum_r x_r @ w_r^T`` (+ residual): this rank's K-shard GEMM with the all-reduce done in its epilogue.

        One-shot (every partial tile pushed to every peer) for small outputs and 2 ranks; two-shot (partials to
        the tile's owner, reduced tile back to everyone) otherwise - then the result lives in the symmetric
        buffer and stays valid until the call after next."""
        from ..ops import gemm

        t, k = x.shape
        n = w.n
        bn = gemm._bn(t)
        tiles = ((n + 127) // 128) * ((t + bn - 1) // bn)
        if self.world == 1 or self.degraded or t * n > self.slot_elems or tiles > 4096 or n % 8:
            return self.all_reduce(gemm.linear(x, w, residual=None)) if residual is None else \
                self.all_reduce(gemm.linear(x, w)).add_(residual)
        if two_shot is None and self.world > 4 and t > 64:
            # measured at 8 ranks (8192 x 5120, K/rank 2176): fused two-shot 1.17 ms, GEMM + NCCL 0.77 ms - the
            # epilogue's remote stores are latency-bound at this fan-out, so the library ring wins until they are
            # replaced by bulk asynchronous copies
            y = TPComm.all_reduce(self, gemm.linear(x, w))
            return y if residual is None else y.add_(residual)
        if two_shot is None:
            two_shot = self.world > 2 and t > 64
        L = _lib.lib()
        if two_shot:
            idx = self._result_index
            self._result_index ^= 1
            rc = L.b200_gemm_wdec_allreduce2(w.wfmt, _lib.ptr(w.weight), _lib.ptr(w.scales), _lib.ptr(x),
                                             _lib.ptr(residual), t, n, k, self._cref(), idx,
                                             ctypes.c_ulonglong(self.budget_ns), _lib.ptr(_lib.status_word(x.device)),
                                             _lib.stream())
            _lib.check(rc, "gemm_wdec_allreduce2")
            self.fused_calls += 1
            return self._result_view(idx, t, n)
        out = torch.empty(t, n, dtype=torch.bfloat16, device=x.device)
        rc = L.b200_gemm_wdec_allreduce(w.wfmt, _lib.ptr(w.weight), _lib.ptr(w.scales), _lib.ptr(x),
                                        _lib.ptr(out), _lib.ptr(residual), t, n, k, self._cref(),
                                        ctypes.c_ulonglong(self.budget_ns),
                                        _lib.ptr(_lib.status_word(x.device)), _lib.stream())
        _lib.check(rc, "gemm_wdec_allreduce")
        self.fused_calls += 1
        return out

    STREAM_FUSED_MAX_T = 8

    def stream_allreduce(self, x: torch.Tensor | None, w, xsplit=None, residual: torch.Tensor | None = None) -> torch.Tensor:
        """Row-parallel decode projection (T <= 32, FP8 weights) with the one-shot all-reduce in the epilogue of the
        weight-streaming GEMM (csrc/kernels/gemm_w8a8s.cu): one launch instead of GEMM + all-reduce kernel."""
        from ..ops import gemm

        t = (xsplit[1].numel() if xsplit is not None else x.shape[0])
        # Measured at 2 ranks (27B shape): one token 7.11 ms/step fused vs 7.10 with the stand-alone all-reduce kernel
        # (two launches fewer per layer, the flag round trip now inside the GEMM's tail); 32 tokens 16.4 vs 13.3 ms -
        # the epilogue owns one feature per thread, so its peer stores are 2 bytes wide, and a 32-token tile pays for
        # that.  Wider batches therefore keep GEMM + vectorised all-reduce.
        if self.world == 1 or self.degraded or t * w.n > self.slot_elems or t > self.STREAM_FUSED_MAX_T:
            y = gemm.linear_stream(x, w, xsplit=xsplit)
            y = self.all_reduce(y)
            return y if residual is None else y.add_(residual)
        return gemm.linear_stream(x, w, residual=residual, xsplit=xsplit, comm=self)

    # ---- sequence-parallel residual stream (csrc/comm/sp_comm.cu, gemm_wdec_kernel.cuh ar_mode 3 / ag_wait)
    SP_FLAG_ROWS = 8

    def sp_rows(self, t: int, h: int) -> int:
        """Rows of the residual stream each rank owns when a ``t``-token chunk runs sequence-parallel, 0 when this
        shape cannot (the shard must be a whole number of 128-token GEMM tiles and the gathered tensor must fit)."""
        if self.world <= 1 or not self.sp_enabled or self.degraded or t % self.world:
            return 0
        rows = t // self.world
        if rows % 128 or t * h > self.slot_elems or h % 8:
            return 0
        return rows

    def linear_rs(self, x: torch.Tensor, w) -> None:
        """Row-parallel GEMM whose epilogue pushes every partial tile to the rank that owns those token rows (the
        push half of a reduce-scatter).  No local result: ``reduce_norm_gather`` on the owner sums the partials."""
        from ..ops import gemm

        t, k = x.shape
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and k == w.k and w.n % 8 == 0
        if w.wfmt == gemm.WF_FP8_B128 and t >= gemm.PREDECODE_MIN_T and w.n % 128 == 0 and k % 64 == 0:
            w = gemm._expanded_bf16(w, x.device)
        bn = ctypes.c_int(0)
        rc = _lib.lib().b200_gemm_wdec_rs(w.wfmt, _lib.ptr(w.weight), _lib.ptr(w.scales), _lib.ptr(x), t, w.n, k,
                                          self._cref(), ctypes.c_ulonglong(self.budget_ns), ctypes.byref(bn),
                                          _lib.ptr(_lib.status_word(x.device)), _lib.stream())
        _lib.check(rc, "gemm_wdec_rs")
        self._rs_bn = bn.value
        self.fused_calls += 1
        self.bytes_reduced += t * w.n * 2

    def reduce_norm_gather(self, h_shard: torch.Tensor, gamma: torch.Tensor | None, eps: float,
                           unit_offset: bool = True, with_partials: bool = True, gather: bool = True) -> torch.Tensor | None:
        """Owner side of the reduce-scatter fused with the residual add, the RMSNorm and the all-gather: sums the
        partials of the last ``linear_rs`` into ``h_shard`` (in place), normalises and stores the rows into every
        rank's gathered buffer.  Returns that buffer, bf16 [world * rows, H]: rows of other ranks become valid as
        their flags arrive (``linear_ag`` waits per tile; anything else calls ``wait_gather`` first)."""
        rows, h = h_shard.shape
        assert h_shard.dtype == torch.bfloat16 and h_shard.is_contiguous()
        L = _lib.lib()
        st = _lib.ptr(_lib.status_word(h_shard.device))
        if self._push_done is not None:
            # the previous push reads the rows this call is about to rewrite
            torch.cuda.current_stream().wait_event(self._push_done)
            self._push_done = None
        deferred = gather and gamma is not None and self.overlap_gather and self.world > 1
        word = -1
        if deferred:
            word = self._epoch_word
            self._epoch_word = (word + 1) & 3
        rc = L.b200_sp_reduce_norm_gather(self._cref(), _lib.ptr(h_shard), _lib.ptr(gamma), ctypes.c_float(eps),
                                          int(unit_offset), rows, h, int(with_partials), self._rs_bn, 0,
                                          int(gather and not deferred), word, st, ctypes.c_ulonglong(self.budget_ns),
                                          _lib.stream())
        _lib.check(rc, "sp_reduce_norm_gather")
        self.fused_calls += 1
        if deferred:
            # the rows are in this rank's own buffer; a second stream pushes them to the peers and raises their flags
            # while the caller's next GEMM starts on the own rows
            if self._side_stream is None:
                self._side_stream = torch.cuda.Stream(device=self.device)
            ready = torch.cuda.Event()
            ready.record()
            self._side_stream.wait_event(ready)
            with torch.cuda.stream(self._side_stream):
                rc = L.b200_sp_push_rows(self._cref(), rows, h, 0, word, _lib.stream())
                _lib.check(rc, "sp_push_rows")
                self._push_done = torch.cuda.Event()
                self._push_done.record()
        return self._result_view(0, rows * self.world, h) if gamma is not None else None

    def linear_ag(self, x_full: torch.Tensor, w, out: torch.Tensor | None = None) -> torch.Tensor:
        """Column-parallel GEMM on the gathered buffer: each token tile is loaded (from local memory) once the rank
        that owns those rows has raised their flags; own rows first."""
        from ..ops import gemm

        t, k = x_full.shape
        assert k == w.k
        if w.wfmt == gemm.WF_FP8_B128 and t >= gemm.PREDECODE_MIN_T and w.n % 128 == 0 and k % 64 == 0:
            w = gemm._expanded_bf16(w, x_full.device)
        if out is None:
            out = torch.empty(t, w.n, dtype=torch.bfloat16, device=x_full.device)
        rc = _lib.lib().b200_gemm_wdec_ag(w.wfmt, _lib.ptr(w.weight), _lib.ptr(w.scales), _lib.ptr(x_full),
                                          _lib.ptr(out), t, w.n, k, self._cref(), self.SP_FLAG_ROWS,
                                          ctypes.c_ulonglong(self.budget_ns), _lib.ptr(_lib.status_word(x_full.device)),
                                          _lib.stream())
        _lib.check(rc, "gemm_wdec_ag")
        self.fused_calls += 1
        return out

    def linear_ag_swiglu(self, x_full: torch.Tensor, w) -> torch.Tensor:
        """``linear_ag`` for the [gate | up] matrix of a feed-forward block with the SwiGLU applied in the epilogue:
        returns silu(gate) * up [T, I] (see ``ops.gemm.linear_swiglu``)."""
        from ..ops import gemm

        out = gemm.linear_swiglu(x_full, w, self._cref(), self.SP_FLAG_ROWS, self.budget_ns)
        self.fused_calls += 1
        return out

    def wait_gather(self, rows: int) -> None:
        """Hold the stream until every peer's rows of the last gather are in this rank's buffer."""
        rc = _lib.lib().b200_sp_wait_gather(self._cref(), rows, _lib.ptr(_lib.status_word(self.device)),
                                            ctypes.c_ulonglong(self.budget_ns), _lib.stream())
        _lib.check(rc, "sp_wait_gather")

    def _ctrl_view(self) -> torch.Tensor:
        """int32 view of this rank's control words ([0] = epoch of the last finished collective, [1] = exit counter)."""
        ptr = int(self.c.ctrl)

        class _Mem:
            __cuda_array_interface__ = {"shape": (16,), "typestr": "<i4", "data": (ptr, False), "version": 2}

        return torch.as_tensor(_Mem(), device=self.device)

    def recover(self, degrade: bool = True) -> None:
        """Collective (every rank of the group calls it once): bring the communicator back to a defined state after a
        bounded wait expired somewhere (``CollectiveTimeoutError``).  The ranks meet on the process group, agree on an
        epoch above every value any of them has used (stale flags and slots then belong to the past), clear the exit
        counter and the error word.  With ``degrade`` the communicator afterwards sends every collective through the
        process group - the step is finished on the library path, as the reference does when its custom all-reduce
        times out (src/models/deepseek_v4/runtime.py:262-268, 4211-4217) - otherwise the peer-memory kernels stay on."""
        torch.cuda.synchronize()
        ctrl = self._ctrl_view()
        top = ctrl[:1].clone().to(torch.int64)
        if self.group is not None or dist.is_initialized():
            dist.all_reduce(top, op=dist.ReduceOp.MAX, group=self.group)
        ctrl[0] = (top[0] + 2).to(torch.int32)
        ctrl[1] = 0
        _lib.status_word(self.device).zero_()
        torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier(group=self.group)
        self.degraded = self.degraded or degrade
        self.recoveries += 1

    def check(self) -> None:
        try:
            _lib.check_status(self.device)
        except _lib.KernelError as e:
            if "peer flag" in str(e):
                raise CollectiveTimeoutError(str(e)) from e
            raise

    def close(self) -> None:
        L = _lib.lib()
        self._push_done = None
        torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier(group=self.group)
        problems = self.verify_guards()
        for p in self._peers:
            L.b200_comm_ipc_close(p)
        self._peers = []
        if self._base is not None:
            L.b200_comm_free(self._base)
            self._base = None
        if problems:
            raise RuntimeError("guard bands disturbed: " + "; ".join(problems))
