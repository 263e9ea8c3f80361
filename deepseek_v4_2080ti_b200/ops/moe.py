"""Routed-expert MoE on the GPU: router top-k, device-side planning, grouped tcgen05 GEMMs over expert-sorted rows
(csrc/kernels/moe.cu + the grouped mode of csrc/kernels/gemm_wdec.cu).  No host synchronisation anywhere: the
number of rows per expert only exists on the device."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib, gemm
from .gemm import WF_BF16, WF_FP8_B128

WF_FP4 = 2
SCORE_FN = {"softmax": 0, "sigmoid": 1, "sqrtsoftplus": 2}


def prepack_fp4(packed: torch.Tensor, scale_e8m0: torch.Tensor) -> torch.Tensor:
    """FP4 weight (uint8 [N, K/2] two codes per byte, low nibble first; E8M0 uint8 [N, K/32]) -> the GEMM's
    tile-major layout uint8 [ceil(N/128), K/64, 4352]: per stage 128 rows x 32 code bytes, then 128 x 2 scale bytes."""
    n, kh = packed.shape
    k = kh * 2
    assert k % 64 == 0 and scale_e8m0.shape == (n, k // 32)
    npad = (n + 127) // 128 * 128
    if npad != n:
        packed = torch.cat([packed, packed.new_zeros(npad - n, kh)])
        scale_e8m0 = torch.cat([scale_e8m0, scale_e8m0.new_zeros(npad - n, k // 32)])
    codes = packed.view(npad // 128, 128, k // 64, 32).permute(0, 2, 1, 3).reshape(npad // 128, k // 64, 128 * 32)
    sc = scale_e8m0.view(npad // 128, 128, k // 64, 2).permute(0, 2, 1, 3).reshape(npad // 128, k // 64, 128 * 2)
    return torch.cat([codes, sc], -1).contiguous()


@dataclass
class ExpertWeights:
    """Stacked weights of this rank's experts for one grouped GEMM."""
    wfmt: int
    weight: torch.Tensor            # fp4/fp8: uint8 [E, mt, kb, stage_bytes]; bf16: [E*N, K]
    scales: torch.Tensor | None     # fp8: fp32 [E, ceil(N/128), K/128]
    n: int
    k: int
    experts: int

    @staticmethod
    def from_fp4(packed: list[torch.Tensor], scales: list[torch.Tensor]) -> "ExpertWeights":
        n, kh = packed[0].shape
        w = torch.stack([prepack_fp4(p, s) for p, s in zip(packed, scales)])
        return ExpertWeights(WF_FP4, w, None, n, kh * 2, len(packed))

    @staticmethod
    def from_fp8(ws: list[torch.Tensor], scales: list[torch.Tensor]) -> "ExpertWeights":
        n, k = ws[0].shape
        w = torch.stack([gemm.prepack_fp8(x) for x in ws])
        return ExpertWeights(WF_FP8_B128, w, torch.stack([s.float() for s in scales]).contiguous(), n, k, len(ws))

    @staticmethod
    def from_gguf(raws: list[torch.Tensor], ggml_type, n: int, k: int) -> "ExpertWeights":
        """Raw GGUF blocks (uint8 [N, row_bytes]) of each expert -> stage-major stacks decoded inside the grouped GEMM.
        ``scales`` carries the codebook table for the formats that need one."""
        from . import gguf_gemm
        w = torch.stack([gguf_gemm.prepack(r, ggml_type, k) for r in raws])
        lut = gguf_gemm.lut_for(ggml_type, raws[0].device)
        return ExpertWeights(gguf_gemm.WF[gguf_gemm.GGMLType(ggml_type)], w, lut, n, k, len(raws))

    @staticmethod
    def from_bf16(ws: list[torch.Tensor]) -> "ExpertWeights":
        n, k = ws[0].shape
        assert n % 128 == 0, "bf16 expert matrices need a multiple of 128 output features"
        return ExpertWeights(WF_BF16, torch.cat([x.to(torch.bfloat16) for x in ws]).contiguous(), None, n, k, len(ws))


def route(logits: torch.Tensor, bias: torch.Tensor | None, k: int, score_func: str, norm_topk: bool,
          route_scale: float) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 logits [T, E] -> (idx int32 [T, k], weights fp32 [T, k])."""
    t, e = logits.shape
    idx = torch.empty(t, k, dtype=torch.int32, device=logits.device)
    wts = torch.empty(t, k, dtype=torch.float32, device=logits.device)
    rc = _lib.lib().b200_moe_route(_lib.ptr(logits), _lib.ptr(bias), t, e, k, SCORE_FN[score_func], int(norm_topk),
                                   ctypes.c_float(route_scale), _lib.ptr(idx), _lib.ptr(wts), _lib.stream())
    _lib.check(rc, "moe_route")
    return idx, wts


def experts_forward(x: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, w13: ExpertWeights, w2: ExpertWeights,
                    expert_lo: int, swiglu_limit: float = 0.0, base: torch.Tensor | None = None, comm=None,
                    residual: torch.Tensor | None = None, comm_mode: int = 0) -> torch.Tensor:
    """out[t] = base[t] + sum_k wts[t,k] * Expert_{idx[t,k]}(x[t]) over the experts [expert_lo, expert_lo + E) held here.
    x [T, H] bf16; w13: [E] x [2I, H] (gate rows then up rows); w2: [E] x [H, I].

    With ``comm`` (a peer-memory communicator of an expert-parallel group) the weighted combine, the sum over ranks
    and the residual add run as one kernel over NVLink (``PeerComm.moe_combine``): every rank gets
    ``residual + sum_ranks(base_r + local routes)``."""
    L0 = _lib.lib()
    t, h = x.shape
    k = idx.shape[1]
    el = w13.experts
    inter = w13.n // 2
    r = t * k
    dev = x.device
    bn = gemm._bn(min(256, max(16, (r + el - 1) // el)))      # token tile sized for the average rows per expert
    if w13.wfmt >= 3:
        bn = min(bn, int(L0.b200_gguf_max_bn(w13.wfmt)), int(L0.b200_gguf_max_bn(w2.wfmt)))
    mt13, mt2 = (w13.n + 127) // 128, (w2.n + 127) // 128
    max_work = (mt13 + mt2) * ((r + bn - 1) // bn + el)
    i32 = lambda *s: torch.empty(*s, dtype=torch.int32, device=dev)
    offsets, route_row, row_token = i32(el + 1), i32(r), i32(r)
    work13, work2 = i32(max_work, 4), i32(max_work, 4)
    n13, n2 = i32(1), i32(1)
    L = _lib.lib()
    s = _lib.stream()
    rc = L.b200_moe_plan(_lib.ptr(idx), t, k, expert_lo, expert_lo + el, _lib.ptr(offsets), _lib.ptr(route_row),
                         _lib.ptr(row_token), _lib.ptr(work13), _lib.ptr(n13), mt13, bn, _lib.ptr(work2), _lib.ptr(n2),
                         mt2, bn, max_work, s)
    _lib.check(rc, "moe_plan")
    # rows past the real count are never read: sized for the worst case (every route local)
    xs = torch.empty(r, h, dtype=torch.bfloat16, device=dev)
    rc = L.b200_moe_gather(_lib.ptr(x), _lib.ptr(row_token), _lib.ptr(offsets), el, _lib.ptr(xs), r, h, s)
    _lib.check(rc, "moe_gather")
    st = _lib.status_word(dev)
    gu = torch.empty(r, w13.n, dtype=torch.bfloat16, device=dev)
    rc = L.b200_gemm_wdec_grouped(w13.wfmt, _lib.ptr(w13.weight), _lib.ptr(w13.scales), _lib.ptr(xs), _lib.ptr(gu), r,
                                  w13.n, w13.k, el, _lib.ptr(work13), _lib.ptr(n13), bn, _lib.ptr(st), s) if w13.wfmt < 3 else \
        L.b200_gemm_wdec_gguf_grouped(w13.wfmt, _lib.ptr(w13.weight), _lib.ptr(w13.scales), _lib.ptr(xs), _lib.ptr(gu), r,
                                      w13.n, w13.k, el, _lib.ptr(work13), _lib.ptr(n13), bn, _lib.ptr(st), s)
    _lib.check(rc, "grouped gemm w13")
    act = torch.empty(r, inter, dtype=torch.bfloat16, device=dev)
    rc = L.b200_moe_swiglu(_lib.ptr(gu), _lib.ptr(offsets), el, _lib.ptr(act), r, inter, ctypes.c_float(swiglu_limit), s)
    _lib.check(rc, "moe_swiglu")
    y = torch.empty(r, h, dtype=torch.bfloat16, device=dev)
    rc = L.b200_gemm_wdec_grouped(w2.wfmt, _lib.ptr(w2.weight), _lib.ptr(w2.scales), _lib.ptr(act), _lib.ptr(y), r, w2.n,
                                  w2.k, el, _lib.ptr(work2), _lib.ptr(n2), bn, _lib.ptr(st), s) if w2.wfmt < 3 else \
        L.b200_gemm_wdec_gguf_grouped(w2.wfmt, _lib.ptr(w2.weight), _lib.ptr(w2.scales), _lib.ptr(act), _lib.ptr(y), r,
                                      w2.n, w2.k, el, _lib.ptr(work2), _lib.ptr(n2), bn, _lib.ptr(st), s)
    _lib.check(rc, "grouped gemm w2")
    if comm is not None and getattr(comm, "world", 1) > 1:
        return comm.moe_combine(y, route_row, wts, base, residual, t, k, h, comm_mode)
    if residual is not None:
        base = residual if base is None else base + residual
    out = torch.empty(t, h, dtype=torch.bfloat16, device=dev)
    rc = L.b200_moe_combine(_lib.ptr(y), _lib.ptr(route_row), _lib.ptr(wts), _lib.ptr(base), _lib.ptr(out), t, k, h, s)
    _lib.check(rc, "moe_combine")
    return out


class OffloadedExperts:
    """Routed experts of one layer kept in pinned host memory with ``capacity`` device slots per matrix
    (``components.expert_cache.HotExpertCache``): a call copies in the experts its tokens route to (least recently
    used ones make room), rewrites the routing ids to slot numbers and runs the ordinary grouped GEMMs over the slot
    arrays.  For models whose experts do not fit beside the caches, and for prefill, where a chunk touches most
    experts once and the copies overlap the previous layer.  A chunk that routes to more experts than there are slots
    is split in halves by tokens.  Reference: GPUPrefillMoEBackend with its hot-expert cache
    (src/components/moe/gpu_prefill_backend.py:41-104, 105-901)."""

    def __init__(self, w13: ExpertWeights, w2: ExpertWeights, capacity: int, device, expert_lo: int = 0):
        from ..components.expert_cache import HotExpertCache
        assert w13.experts == w2.experts and (w13.scales is None or w13.wfmt >= 3) and (w2.scales is None or w2.wfmt >= 3), \
            "per-expert scale grids (FP8) are not packed into the slabs"
        self.experts, self.expert_lo = w13.experts, int(expert_lo)
        self.capacity = min(int(capacity), self.experts)
        self.dev = torch.device(device)

        def split(w: ExpertWeights):
            per = w.weight.reshape(w.experts, -1)
            host = per.contiguous().view(torch.uint8).cpu()
            cache = HotExpertCache(host, self.capacity, self.dev)
            shape = (self.capacity * w.n, w.k) if w.wfmt == WF_BF16 else (self.capacity, *w.weight.shape[1:])
            view = cache.slots.view(w.weight.dtype).view(*shape)
            lut = w.scales.to(self.dev) if w.scales is not None else None
            return cache, ExpertWeights(w.wfmt, view, lut, w.n, w.k, self.capacity)

        self.c13, self.w13 = split(w13)
        self.c2, self.w2 = split(w2)

    def stats(self) -> dict:
        a, b = self.c13.stats, self.c2.stats
        return {"hits": a.hits + b.hits, "misses": a.misses + b.misses, "evictions": a.evictions + b.evictions,
                "bytes_copied": a.bytes_copied + b.bytes_copied}

    def forward(self, x: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, swiglu_limit: float = 0.0,
                base: torch.Tensor | None = None) -> torch.Tensor:
        lo, hi = self.expert_lo, self.expert_lo + self.experts
        local = (idx >= lo) & (idx < hi)
        need = torch.unique(idx[local]).tolist()                       # host sync: the copies depend on the routing
        if len(need) > self.capacity and x.shape[0] > 1:
            h = x.shape[0] // 2
            parts = [self.forward(x[a:b].contiguous(), idx[a:b].contiguous(), wts[a:b].contiguous(), swiglu_limit,
                                  None if base is None else base[a:b].contiguous()) for a, b in ((0, h), (h, x.shape[0]))]
            return torch.cat(parts)
        if len(need) > self.capacity:
            raise RuntimeError(f"one token routes to {len(need)} experts of this rank; the cache holds {self.capacity}")
        local_ids = [e - lo for e in need]
        s13, s2 = self.c13.fetch(local_ids), self.c2.fetch(local_ids)
        assert torch.equal(s13, s2), "the two caches see the same requests and must agree on the slots"
        table = torch.full((self.experts + 1,), self.capacity, dtype=torch.int32, device=idx.device)
        if local_ids:
            table[torch.tensor(local_ids, dtype=torch.long, device=idx.device)] = s13.to(idx.device)
        # ids of other ranks' experts map to `capacity`: outside [0, capacity), so the routing plan drops them
        slot_idx = table[torch.where(local, idx - lo, torch.full_like(idx, self.experts)).long()].contiguous()
        return experts_forward(x, slot_idx, wts, self.w13, self.w2, 0, swiglu_limit, base)
