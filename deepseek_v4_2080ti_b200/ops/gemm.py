"""Weight-decoding tcgen05 GEMM front-end (csrc/kernels/gemm_wdec.cu).

``y[T, N] = x[T, K] @ W[N, K]^T`` with bf16 activations and either bf16 weights or FP8 E4M3
weights carrying one scale per 128x128 block; FP8 weights are decoded inside the kernel.
Covers the reference's FP8 block-128 projections (cpp_engine/backends/cuda/kernels/qwen_half_ops.cu:988-1199)
and bf16 matvec/matmul (cpp_engine/backends/cuda/kernels/bf16_ops.cu:30-167).
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

import torch

from ..utils import canary
from . import _lib

WF_BF16 = 0
WF_FP8_B128 = 1
NUM_SMS = 148


def prepack_fp8(w: torch.Tensor) -> torch.Tensor:
    """FP8 weight [N, K] -> the kernel's tile-major layout [ceil(N/128), ceil(K/64), 128, 64] (uint8).

    Two transformations, both done once at load time:
    * every 4 consecutive bytes (w0,w1,w2,w3) are stored as (w0,w2,w1,w3): the decode warps turn one
      32-bit word into two bf16x2 words with shifts and masks only, and this order makes those words
      come out as (w0,w1) and (w2,w3);
    * each [128 rows x 64 bytes] pipeline-stage tile is contiguous (8 KB), so a stage is fetched with a
      single bulk copy instead of 128 separate 64-byte rows;
    * inside a tile the four 16-byte chunks of row r are stored at chunk index ``c ^ ((r >> 1) & 3)``
      (the 64-byte shared-memory swizzle), so the bulk copy lands in the layout an FP8 tensor-core
      operand descriptor expects and the small-batch kernel can use the bytes without touching them.
    """
    u = w.view(torch.uint8)
    n, k = u.shape
    npad, kpad = (n + 127) // 128 * 128, (k + 63) // 64 * 64
    if (npad, kpad) != (n, k):
        full = torch.zeros(npad, kpad, dtype=torch.uint8, device=u.device)
        full[:n, :k] = u
        u = full
    u = u.view(npad, kpad // 4, 4)[:, :, [0, 2, 1, 3]].reshape(npad // 128, 128, kpad // 64, 64)
    u = u.permute(0, 2, 1, 3).contiguous()                       # [mt, kb, 128 rows, 64 bytes]
    # 64-byte swizzle: 16-byte chunk c of row r is stored at chunk c ^ ((r >> 1) & 3)
    r = torch.arange(128, device=u.device)
    c = torch.arange(4, device=u.device)
    src_chunk = c[None, :] ^ ((r[:, None] >> 1) & 3)             # physical chunk p holds logical chunk p ^ s
    idx = (src_chunk[:, :, None] * 16 + torch.arange(16, device=u.device)[None, None, :]).reshape(128, 64)
    return torch.gather(u, 3, idx[None, None].expand(u.shape[0], u.shape[1], 128, 64)).contiguous()


@dataclass
class PackedLinear:
    """A weight matrix as the GEMM kernel consumes it."""
    wfmt: int
    weight: torch.Tensor          # uint8 [N, K] (prepacked fp8) or bf16 [N, K]
    scales: torch.Tensor | None   # fp32 [ceil(N/128), ceil(K/128)]
    n: int
    k: int

    @staticmethod
    def from_fp8(w_fp8: torch.Tensor, scale: torch.Tensor) -> "PackedLinear":
        n, k = w_fp8.shape
        return PackedLinear(WF_FP8_B128, prepack_fp8(w_fp8), scale.float().contiguous(), n, k)

    @staticmethod
    def from_bf16(w: torch.Tensor) -> "PackedLinear":
        n, k = w.shape
        return PackedLinear(WF_BF16, w.to(torch.bfloat16).contiguous(), None, n, k)

    def nbytes(self) -> int:
        return self.weight.numel() * self.weight.element_size() + (0 if self.scales is None else self.scales.numel() * 4)


_workspaces: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
MAX_TILE_COUNTERS = 1 << 16


def _workspace(nfloats: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    """(fp32 split-K scratch, zeroed int32 tile counters) of the device; grown on demand, never shrunk.
    The kernel leaves the counters at zero, so they are cleared only when allocated."""
    key = torch.device(device).index or 0
    ws = _workspaces.get(key)
    if ws is None or ws[0].numel() < nfloats:
        ws = (canary.empty(max(nfloats, 1 << 22), dtype=torch.float32, device=device, name="gemm split-K partials"),
              ws[1] if ws is not None else canary.zeros(MAX_TILE_COUNTERS, dtype=torch.int32, device=device,
                                                        name="gemm tile counters"))
        _workspaces[key] = ws
    return ws


PREDECODE_MIN_T = 2048


class _Expander:
    """Two bf16 scratch buffers per device for FP8 matrices expanded ahead of a prefill-sized GEMM.  ``prefetch`` runs
    the expansion of the NEXT matrix on a side stream while the current GEMM (tensor-bound, few registers, no spare
    shared memory but spare threads) runs on the main one: the expansion is a pure HBM pass and hides under it.
    A buffer is rewritten only after the GEMM that last read it: the side stream waits for an event recorded on the
    main stream at prefetch time, which is after that GEMM's launch and before the launch of the GEMM it overlaps."""

    def __init__(self, device):
        self.device = device
        self.bufs: list[torch.Tensor | None] = [None, None]
        self.tags: list[tuple | None] = [None, None]
        self.ready: list[torch.cuda.Event | None] = [None, None]
        self.turn = 0
        self.side: torch.cuda.Stream | None = None

    def _slot(self, need: int, keep: tuple | None = None) -> int:
        """A buffer that holds no pending expansion (never the one tagged ``keep``); both free: take turns."""
        free = [i for i in (0, 1) if self.tags[i] is None]
        if len(free) == 1:
            s = free[0]
        else:
            s = self.turn
            if keep is not None and self.tags[s] == keep:
                s ^= 1
        self.turn = s ^ 1
        buf = self.bufs[s]
        if buf is None or buf.numel() < need:
            self.bufs[s] = canary.empty(max(need, 1 << 26), dtype=torch.bfloat16, device=self.device,
                                        name=f"fp8 expansion buffer {s}")
        return s

    @staticmethod
    def _key(w: "PackedLinear", gate_up: bool = False) -> tuple:
        return (w.weight.data_ptr(), w.n, w.k, gate_up)

    def _unpack(self, w: "PackedLinear", s: int, gate_up: bool = False) -> torch.Tensor:
        out = self.bufs[s][:w.n * w.k].view(w.n, w.k)
        fn = _lib.lib().b200_unpack_fp8_bf16_gate_up if gate_up else _lib.lib().b200_unpack_fp8_bf16
        rc = fn(_lib.ptr(w.weight), _lib.ptr(w.scales), _lib.ptr(out), w.n, w.k, _lib.stream())
        _lib.check(rc, "unpack_fp8_bf16")
        return out

    def prefetch(self, w: "PackedLinear", current: "PackedLinear | None" = None, gate_up: bool = False) -> None:
        """``current``: the matrix of the GEMM that is about to be launched (its buffer must survive).  ``gate_up``:
        write the rows interleaved for the SwiGLU epilogue (``linear_swiglu``)."""
        key = self._key(w, gate_up)
        if key in self.tags:
            return
        main = torch.cuda.current_stream(self.device)
        if self.side is None:
            self.side = torch.cuda.Stream(self.device)
        keep = None
        if current is not None:
            keep = next((t for t in self.tags if t is not None and t[:3] == self._key(current)[:3]), None)
        s = self._slot(w.n * w.k, keep)
        if self.ready[s] is not None:                 # an expansion nobody used is still writing this buffer
            self.side.wait_event(self.ready[s])
        # everything launched on the main stream so far, the last reader of this buffer included, comes first; a
        # buffer allocated just now was allocated on the main stream, so the wait also orders its first use
        self.side.wait_event(main.record_event())
        with torch.cuda.stream(self.side):
            self._unpack(w, s, gate_up)
            self.ready[s] = self.side.record_event()
        self.tags[s] = key

    def get(self, w: "PackedLinear", gate_up: bool = False) -> torch.Tensor:
        key = self._key(w, gate_up)
        main = torch.cuda.current_stream(self.device)
        if key in self.tags:
            s = self.tags.index(key)
            if self.ready[s] is not None:
                main.wait_event(self.ready[s])
                self.ready[s] = None
            self.tags[s] = None                       # good for this one GEMM; the next prefetch but one may reuse it
            self.turn = s ^ 1
            return self.bufs[s][:w.n * w.k].view(w.n, w.k)
        s = self._slot(w.n * w.k)
        if self.ready[s] is not None:
            main.wait_event(self.ready[s])
            self.ready[s] = None
        self.tags[s] = None
        return self._unpack(w, s, gate_up)


_expanders: dict[int, _Expander] = {}


def _expander(device) -> _Expander:
    key = torch.device(device).index or 0
    e = _expanders.get(key)
    if e is None:
        e = _expanders[key] = _Expander(torch.device("cuda", key))
    return e


def prefetch_bf16(w: "PackedLinear | None", device, current: "PackedLinear | None" = None, gate_up: bool = False) -> None:
    """Start expanding FP8 matrix ``w`` to bf16 on the side stream; the next prefill-sized ``linear`` on ``w`` picks
    the result up instead of expanding on its own stream.  Call it right BEFORE launching the GEMM on ``current``, the
    one it is meant to overlap.  No-op for other formats."""
    if w is not None and w.wfmt == WF_FP8_B128 and os.environ.get("B200_EXPAND_PREFETCH", "1") != "0":
        _expander(device).prefetch(w, current, gate_up)


def _expanded_bf16(w: "PackedLinear", device, gate_up: bool = False) -> "PackedLinear":
    """bf16 copy of an FP8 block-128 matrix in a per-device scratch buffer (valid until the next two expansions)."""
    return PackedLinear(WF_BF16, _expander(device).get(w, gate_up), None, w.n, w.k)


def swiglu_fusable(t: int, w: "PackedLinear") -> bool:
    """Can ``linear_swiglu`` take [gate | up] matrix ``w`` for ``t`` tokens?  FP8 weights (they are re-laid-out while
    being expanded), a prefill-sized batch, and a shape the CTA-pair kernel tiles evenly."""
    return (w.wfmt == WF_FP8_B128 and t >= PREDECODE_MIN_T and w.n % 256 == 0 and w.k % 64 == 0 and
            os.environ.get("B200_SWIGLU_FUSED", "1") != "0" and
            bool(_lib.lib().b200_gemm_2cta_supported(t, w.n, w.k)))


def linear_swiglu(x: torch.Tensor, w: "PackedLinear", comm_ref=None, flag_rows: int = 0, budget_ns: int = 0,
                  out: torch.Tensor | None = None) -> torch.Tensor:
    """``silu(x @ gate^T) * (x @ up^T)`` for ``w = [gate | up]`` ([2I, K]) in ONE kernel: the weights are expanded
    with gate and up tiles interleaved and the activation is applied to the fp32 accumulators in the GEMM epilogue
    (no [T, 2I] intermediate).  ``comm_ref``: ctypes reference of a ``B200Comm`` when ``x`` is the gathered buffer of
    the sequence-parallel path.  Reference behaviour: cpp_engine's mlp gate_up GEMM followed by ``silu_mul``
    (cpp_engine/backends/cuda/kernels/qwen_half_ops.cu:2730-2745)."""
    t, k = x.shape
    assert swiglu_fusable(t, w) and k == w.k and x.dtype == torch.bfloat16 and x.is_contiguous()
    wb = _expanded_bf16(w, x.device, gate_up=True)
    if out is None:
        out = torch.empty(t, w.n // 2, dtype=torch.bfloat16, device=x.device)
    rc = _lib.lib().b200_gemm_bf16_swiglu(_lib.ptr(wb.weight), _lib.ptr(x), _lib.ptr(out), t, w.n, k, comm_ref, flag_rows,
                                          ctypes.c_ulonglong(budget_ns), _lib.ptr(_lib.status_word(x.device)), _lib.stream())
    _lib.check(rc, "gemm_bf16_swiglu")
    return out


def _bn(t: int) -> int:
    return 16 if t <= 16 else 32 if t <= 32 else 64 if t <= 64 else 128 if t <= 128 else 256


def pick_splits(t: int, n: int, k: int) -> int:
    """Split K when the tile grid alone cannot fill the 148 SMs evenly (small-batch decode).

    The persistent grid runs ceil(units / 148) waves of (tile, split) units; the split count that wastes
    the least of the last wave wins, subject to at least 8 k-blocks (512 columns) per split so the
    pipeline fill is amortised, and to a bound on the fp32 partial traffic for larger T."""
    if t > 128:
        return 1
    tiles = ((n + 127) // 128) * ((t + _bn(t) - 1) // _bn(t))
    kb = (k + 63) // 64
    max_s = max(1, min(kb // 8, 16 if t <= 16 else 8 if t <= 64 else 4))
    best, best_eff = 1, 0.0
    for s in range(1, max_s + 1):
        per = (kb + s - 1) // s
        s_eff = (kb + per - 1) // per
        if s_eff != s:
            continue
        units = tiles * s
        waves = (units + NUM_SMS - 1) // NUM_SMS
        # the longest split sets the pace of a wave
        eff = (tiles * kb) / (waves * NUM_SMS * per)
        if eff > best_eff + 0.02:
            best, best_eff = s, eff
    return best


STREAM_MAX_T = 32   # token counts served by the weight-streaming FP8 kernel (csrc/kernels/gemm_w8a8s.cu)


def stream_layout(t: int) -> tuple[int, int]:
    """(MMA N, number of E4M3 terms per activation) the streaming kernel uses for ``t`` tokens."""
    if t <= 5:
        return 16, 3
    if t <= 8:
        return 16, 2
    if t <= 16:
        return 32, 2
    return 64, 2


def pick_splits_stream(n: int, k: int) -> int:
    """Split count for the streaming kernel: units are (128-row tile, run of 128-wide K blocks).
    Every unit ends with a fix-up (fence, counter, reduction by the last arriver), so the smallest
    split count that fills at least 85% of the waves wins; more splits only when they gain > 5%."""
    tiles = (n + 127) // 128
    kblk = k // 128
    best, best_eff = 1, 0.0
    for s in range(1, max(1, min(kblk // 4, 16)) + 1):
        per = (kblk + s - 1) // s
        if (kblk + per - 1) // per != s:
            continue
        waves = (tiles * s + NUM_SMS - 1) // NUM_SMS
        eff = (tiles * kblk) / (waves * NUM_SMS * per)
        if eff > best_eff + 0.05:
            best, best_eff = s, eff
        if best_eff >= 0.85:
            break
    return best


def split_activations(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16 [T, K] -> (uint8 [T*terms, K] E4M3 terms, fp32 [T] inverse row scales) for ``linear_stream``."""
    t, k = x.shape
    _, terms = stream_layout(t)
    xq = torch.empty(t * terms, k, dtype=torch.uint8, device=x.device)
    inv_c = torch.empty(t, dtype=torch.float32, device=x.device)
    rc = _lib.lib().b200_act_split_e4m3(_lib.ptr(x), t, k, terms, _lib.ptr(xq), _lib.ptr(inv_c), _lib.stream())
    _lib.check(rc, "act_split_e4m3")
    return xq, inv_c


def linear_stream(x: torch.Tensor, w: PackedLinear, residual: torch.Tensor | None = None,
                  out: torch.Tensor | None = None, splits: int | None = None,
                  xsplit: tuple[torch.Tensor, torch.Tensor] | None = None, comm=None) -> torch.Tensor:
    """Small-batch (T <= 32) FP8 projection: weights go from HBM to the tensor core untouched, the
    activations are split into E4M3 terms instead.  ``xsplit`` reuses a previous ``split_activations(x)``.
    ``comm`` (a ``parallel.tp.PeerComm``): row-parallel form, the one-shot all-reduce over the ranks happens in the
    epilogue (sum over ranks + residual in ``out`` on every rank)."""
    xq, inv_c = xsplit if xsplit is not None else split_activations(x)
    t, k = inv_c.numel(), xq.shape[1]        # x itself may be None when the split is supplied
    n = w.n
    dev = xq.device
    assert w.wfmt == WF_FP8_B128 and t <= STREAM_MAX_T and k % 128 == 0 and k == w.k
    if out is None:
        out = torch.empty(t, n, dtype=torch.bfloat16, device=dev)
    if splits is None:
        splits = pick_splits_stream(n, k)
    kblk = k // 128
    splits = max(1, min(splits, kblk))
    per = (kblk + splits - 1) // splits
    splits = (kblk + per - 1) // per
    if (n + 127) // 128 > MAX_TILE_COUNTERS:
        splits = 1
    ws, counters = _workspace(splits * t * n, dev) if splits > 1 else (None, None)
    if comm is not None:
        rc = _lib.lib().b200_gemm_w8a8s_allreduce(_lib.ptr(w.weight), _lib.ptr(w.scales), _lib.ptr(xq), _lib.ptr(inv_c),
                                                  _lib.ptr(out), _lib.ptr(residual), t, n, k, splits, _lib.ptr(ws),
                                                  _lib.ptr(counters), comm._cref(), ctypes.c_ulonglong(comm.budget_ns),
                                                  _lib.ptr(_lib.status_word(dev)), _lib.stream())
        _lib.check(rc, "gemm_w8a8s_allreduce")
        comm.fused_calls += 1
        return out
    rc = _lib.lib().b200_gemm_w8a8s(_lib.ptr(w.weight), _lib.ptr(w.scales), _lib.ptr(xq), _lib.ptr(inv_c),
                                    _lib.ptr(out), _lib.ptr(residual), t, n, k, splits, _lib.ptr(ws),
                                    _lib.ptr(counters), _lib.ptr(_lib.status_word(dev)), _lib.stream())
    _lib.check(rc, "gemm_w8a8s")
    return out


def linear(x: torch.Tensor, w: PackedLinear, residual: torch.Tensor | None = None,
           out: torch.Tensor | None = None, splits: int | None = None,
           out_f32: bool = False, stream: bool | None = None) -> torch.Tensor:
    """``x [T, K] bf16`` -> ``[T, N]`` bf16 (or fp32 when ``out_f32``).  FP8 weights with T <= 32 go to the
    weight-streaming kernel (``stream=False`` forces the decode-warp kernel); split-K partials are
    reduced inside the kernel by the last-arriving CTA of each output tile."""
    assert x.dtype == torch.bfloat16 and x.is_cuda and x.dim() == 2 and x.is_contiguous()
    t, k = x.shape
    assert k == w.k, (k, w.k)
    n = w.n
    if w.wfmt == WF_FP8_B128 and t <= STREAM_MAX_T and k % 128 == 0 and not out_f32 and stream is not False:
        return linear_stream(x, w, residual, out, splits)
    if w.wfmt == WF_FP8_B128 and t >= PREDECODE_MIN_T and not out_f32 and n % 128 == 0 and k % 64 == 0:
        # prefill-sized batch: every weight tile would be decoded once per 256-token tile of the batch, so the matrix is
        # expanded to bf16 once (one pass over the weights, ~3 % of the GEMM) and multiplied by the bf16 path, which
        # has no decode traffic through shared memory (1.17 / 1.38 PFLOP/s against 1.09 / 1.16 at 8192 x 17408 x 5120
        # and 8192 x 5120 x 17408)
        w = _expanded_bf16(w, x.device)
    if splits is None:
        splits = 1 if out_f32 else pick_splits(t, n, k)
    L = _lib.lib()
    st = _lib.status_word(x.device)
    if out_f32:
        o32 = out if out is not None else torch.empty(t, n, dtype=torch.float32, device=x.device)
        rc = L.b200_gemm_wdec(w.wfmt, _lib.ptr(w.weight), _lib.ptr(w.scales), _lib.ptr(x), None,
                              _lib.ptr(o32), None, t, n, k, 1, _lib.ptr(st), _lib.stream())
        _lib.check(rc, "gemm_wdec")
        return o32
    if out is None:
        out = torch.empty(t, n, dtype=torch.bfloat16, device=x.device)
    kb = (k + 63) // 64
    splits = max(1, min(splits, kb))
    per = (kb + splits - 1) // splits
    splits = (kb + per - 1) // per          # same rule as the launcher: no empty split
    tiles = ((n + 127) // 128) * ((t + _bn(t) - 1) // _bn(t))
    if splits > 1 and tiles > MAX_TILE_COUNTERS:
        splits = 1
    if splits <= 1:
        rc = L.b200_gemm_wdec(w.wfmt, _lib.ptr(w.weight), _lib.ptr(w.scales), _lib.ptr(x), _lib.ptr(out),
                              None, _lib.ptr(residual), t, n, k, 1, _lib.ptr(st), _lib.stream())
        _lib.check(rc, "gemm_wdec")
        return out
    ws, counters = _workspace(splits * t * n, x.device)
    rc = L.b200_gemm_wdec_ex(w.wfmt, _lib.ptr(w.weight), _lib.ptr(w.scales), _lib.ptr(x), _lib.ptr(out),
                             _lib.ptr(ws), _lib.ptr(residual), t, n, k, splits, _lib.ptr(counters),
                             _lib.ptr(st), _lib.stream())
    _lib.check(rc, "gemm_wdec(split-k)")
    return out


def linear_ref(x: torch.Tensor, w_fp32: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 oracle: x @ w^T (+ residual)."""
    y = x.float() @ w_fp32.float().t()
    if residual is not None:
        y = y + residual.float()
    return y
