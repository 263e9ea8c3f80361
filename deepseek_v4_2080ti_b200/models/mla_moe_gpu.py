"""GPU runtime of the MLA + routed-expert family (DeepSeek-V4-Flash-shaped, GLM-5.2-shaped): every op on the forward
path is one of this package's sm_100a kernels.

* projections: weight-decoding tcgen05 GEMM (bf16 or FP8 block-128 weights);
* attention: absorbed MLA over a paged latent cache (``ops/mla.py``): per-head absorption GEMMs run as one grouped
  GEMM, the lightning indexer scores every cached key and a radix top-k picks the keys each query attends to;
* feed-forward: dense SwiGLU for the leading layers, otherwise router top-k -> device-side plan -> grouped FP4 / FP8 /
  bf16 expert GEMMs -> weighted combine on top of the shared expert (``ops/moe.py``);
* parallelism: attention heads and the dense / shared intermediate dimension are sharded over the tensor-parallel
  group, routed experts are sharded by contiguous expert range; partial outputs are summed by ``comm``.

Same math as ``MlaMoeRuntime`` (the host path) and ``reference_cpu/mla_moe_ref.py``; see ``mla_moe.py`` for the
reference citations.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterator

import torch

from ..formats import fp8 as fp8fmt
from ..ops import basic, gemm, mla, moe
from ..ops.gemm import PackedLinear
from .mla_moe import MlaMoeConfig


class _NoComm:
    world, rank = 1, 0

    def all_reduce(self, t):
        return t


@dataclass
class GpuLayer:
    attn_norm: torch.Tensor
    ffn_norm: torch.Tensor
    wq_a: PackedLinear | None
    q_norm: torch.Tensor | None
    wq_b: PackedLinear
    wkv_a: PackedLinear
    kv_norm: torch.Tensor
    w_uk_t: torch.Tensor          # [H_local * C, N] bf16: head h rows hold W_uk[h]^T
    w_uv: torch.Tensor            # [H_local * V, C] bf16
    wo: PackedLinear
    idx_wq: PackedLinear | None = None
    idx_wk: PackedLinear | None = None
    idx_knorm: torch.Tensor | None = None
    idx_wproj: PackedLinear | None = None
    dense_gu: PackedLinear | None = None
    dense_down: PackedLinear | None = None
    gate: PackedLinear | None = None
    gate_bias: torch.Tensor | None = None
    shared_gu: PackedLinear | None = None
    shared_down: PackedLinear | None = None
    w13: moe.ExpertWeights | None = None
    w2: moe.ExpertWeights | None = None


class MlaMoeGpuWeights:
    def __init__(self, cfg: MlaMoeConfig, state: Iterator[tuple[str, torch.Tensor]], device="cuda", rank: int = 0,
                 world: int = 1, dense_fp8: bool = False):
        self.cfg, self.device, self.rank, self.world, self.dense_fp8 = cfg, torch.device(device), rank, world, dense_fp8
        assert cfg.num_heads % world == 0 and cfg.num_experts % world == 0
        self.h_local = cfg.num_heads // world
        per = cfg.num_experts // world
        self.expert_lo, self.expert_hi = rank * per, (rank + 1) * per
        sd: dict[str, torch.Tensor] = {}
        for k, v in state:
            if ".experts." in k:
                e = int(k.split(".experts.")[1].split(".")[0])
                if not (self.expert_lo <= e < self.expert_hi):
                    continue
            sd[k] = v
        dev = self.device
        self.embed = sd["embed.weight"].to(dev, torch.bfloat16).contiguous()
        self.norm = sd["norm.weight"].to(dev, torch.bfloat16)
        self.head = PackedLinear.from_bf16(sd["head.weight"].to(dev))
        self.layers = [self._layer(sd, f"layers.{i}.", i < cfg.first_dense_layers) for i in range(cfg.num_layers)]

    def _lin(self, w: torch.Tensor) -> PackedLinear:
        w = w.to(self.device)
        if self.dense_fp8 and w.shape[0] % 128 == 0 and w.shape[1] % 128 == 0:
            q, s = fp8fmt.quantize_block128(w.float())
            return PackedLinear.from_fp8(q, s)
        return PackedLinear.from_bf16(w)

    def _rows(self, w: torch.Tensor, group: int = 1) -> torch.Tensor:
        """Output-feature shard of a column-parallel matrix (``group`` rows stay together)."""
        n = w.shape[0] // self.world
        assert n * self.world == w.shape[0] and n % group == 0
        return w[self.rank * n:(self.rank + 1) * n]

    def _cols(self, w: torch.Tensor) -> torch.Tensor:
        k = w.shape[1] // self.world
        return w[:, self.rank * k:(self.rank + 1) * k]

    def _layer(self, sd, p: str, dense: bool) -> GpuLayer:
        cfg, dev = self.cfg, self.device
        b = lambda t: t.to(dev, torch.bfloat16).contiguous()
        a = p + "attn."
        hq = cfg.qk_head_dim
        wkv_b = self._rows(sd[a + "wkv_b.weight"], cfg.qk_nope_dim + cfg.v_head_dim).to(dev, torch.bfloat16)
        wkv_b = wkv_b.view(self.h_local, cfg.qk_nope_dim + cfg.v_head_dim, cfg.kv_lora_rank)
        w_uk = wkv_b[:, :cfg.qk_nope_dim]                       # [H, N, C]
        lw = GpuLayer(
            attn_norm=b(sd[p + "attn_norm.weight"]), ffn_norm=b(sd[p + "ffn_norm.weight"]),
            wq_a=self._lin(sd[a + "wq_a.weight"]) if cfg.q_lora_rank > 0 else None,
            q_norm=b(sd[a + "q_norm.weight"]) if cfg.q_lora_rank > 0 else None,
            wq_b=self._lin(self._rows(sd[a + ("wq_b.weight" if cfg.q_lora_rank > 0 else "wq.weight")], hq)),
            wkv_a=self._lin(sd[a + "wkv_a.weight"]), kv_norm=b(sd[a + "kv_norm.weight"]),
            w_uk_t=w_uk.transpose(1, 2).reshape(self.h_local * cfg.kv_lora_rank, cfg.qk_nope_dim).contiguous(),
            w_uv=wkv_b[:, cfg.qk_nope_dim:].reshape(self.h_local * cfg.v_head_dim, cfg.kv_lora_rank).contiguous(),
            wo=self._lin(self._cols(sd[a + "wo.weight"])))
        if cfg.index_heads > 0:
            # the indexer is small and replicated: every rank scores with all index heads
            lw.idx_wq, lw.idx_wk = self._lin(sd[a + "indexer.wq_b.weight"]), self._lin(sd[a + "indexer.wk.weight"])
            lw.idx_knorm, lw.idx_wproj = b(sd[a + "indexer.k_norm.weight"]), self._lin(sd[a + "indexer.weights_proj.weight"])
        f = p + "ffn."
        if dense:
            lw.dense_gu = self._lin(torch.cat([self._rows(sd[f + "w1.weight"]), self._rows(sd[f + "w3.weight"])]))
            lw.dense_down = self._lin(self._cols(sd[f + "w2.weight"]))
            return lw
        lw.gate = PackedLinear.from_bf16(sd[f + "gate.weight"].to(dev))
        lw.gate_bias = sd[f + "gate.bias"].to(dev, torch.float32)
        if cfg.num_shared_experts:
            lw.shared_gu = self._lin(torch.cat([self._rows(sd[f + "shared_experts.w1.weight"]),
                                                self._rows(sd[f + "shared_experts.w3.weight"])]))
            lw.shared_down = self._lin(self._cols(sd[f + "shared_experts.w2.weight"]))
        es = range(self.expert_lo, self.expert_hi)
        if cfg.expert_format == "fp4":
            cat13 = lambda e, suf: torch.cat([sd[f + f"experts.{e}.w1.{suf}"], sd[f + f"experts.{e}.w3.{suf}"]]).to(dev)
            lw.w13 = moe.ExpertWeights.from_fp4([cat13(e, "weight") for e in es], [cat13(e, "scale") for e in es])
            lw.w2 = moe.ExpertWeights.from_fp4([sd[f + f"experts.{e}.w2.weight"].to(dev) for e in es],
                                               [sd[f + f"experts.{e}.w2.scale"].to(dev) for e in es])
        else:
            lw.w13 = moe.ExpertWeights.from_bf16([torch.cat([sd[f + f"experts.{e}.w1.weight"], sd[f + f"experts.{e}.w3.weight"]]).to(dev)
                                                  for e in es])
            lw.w2 = moe.ExpertWeights.from_bf16([sd[f + f"experts.{e}.w2.weight"].to(dev) for e in es])
        return lw


class MlaMoeGpuRuntime:
    """One sequence at a time (prefill in one or more chunks, then token-by-token decode) over a paged latent cache."""

    def __init__(self, cfg: MlaMoeConfig, weights: MlaMoeGpuWeights, max_context: int = 4096, block_size: int = 64, comm=None):
        self.cfg, self.w, self.device = cfg, weights, weights.device
        self.comm = comm or _NoComm()
        self.bs = block_size
        self.max_context = max_context
        nblk = (max_context + block_size - 1) // block_size
        rows = nblk * block_size
        n = cfg.num_layers
        d = cfg.kv_lora_rank + cfg.qk_rope_dim
        self.cache = torch.zeros(n, rows, d, dtype=torch.bfloat16, device=self.device)
        self.idx_cache = torch.zeros(n, rows, max(1, cfg.index_dim), dtype=torch.bfloat16, device=self.device)
        # identity page table: block b of the sequence is physical block b (one resident sequence)
        self.block_table = torch.arange(nblk, dtype=torch.int32, device=self.device).view(1, nblk).contiguous()
        self.length = 0

    def reset(self) -> None:
        self.length = 0

    def _swiglu(self, x, gu: PackedLinear, down: PackedLinear):
        return gemm.linear(basic.silu_mul(gemm.linear(x, gu)), down)

    def _attention(self, lw: GpuLayer, i: int, x: torch.Tensor, pos: torch.Tensor, end: int) -> torch.Tensor:
        cfg = self.cfg
        t = x.shape[0]
        hl = self.w.h_local
        eps = cfg.rms_norm_eps
        qin = basic.rmsnorm(gemm.linear(x, lw.wq_a), lw.q_norm, eps) if lw.wq_a is not None else x
        q = gemm.linear(qin, lw.wq_b)
        kv = gemm.linear(x, lw.wkv_a)
        kidx = gemm.linear(x, lw.idx_wk) if lw.idx_wk is not None else None
        mla.kv_append(kv, lw.kv_norm, eps, pos, pos, cfg.rope_theta, self.cache[i], cfg.kv_lora_rank, cfg.qk_rope_dim,
                      kidx, lw.idx_knorm, self.idx_cache[i] if kidx is not None else None)
        qn_t, q_pe = mla.q_prepare(q, pos, cfg.rope_theta, hl, cfg.qk_nope_dim, cfg.qk_rope_dim)
        q_lat = mla.per_head_linear(qn_t, lw.w_uk_t)
        sel = None
        if lw.idx_wq is not None and end > cfg.index_topk:
            qi = gemm.linear(qin, lw.idx_wq).view(t, cfg.index_heads, cfg.index_dim)
            hw = gemm.linear(x, lw.idx_wproj, out_f32=True) * cfg.index_heads ** -0.5
            scores = mla.indexer_scores(qi, hw.contiguous(), self.idx_cache[i], self.block_table, self.bs, pos, end,
                                        cfg.index_dim ** -0.5)
            sel = mla.topk_rows(scores, (pos + 1).to(torch.int32), cfg.index_topk)
        o_lat = mla.attention(q_lat, q_pe, self.cache[i], self.block_table, self.bs, pos, cfg.kv_lora_rank, cfg.qk_rope_dim,
                              cfg.qk_head_dim ** -0.5, sel)
        o = mla.transpose_heads(mla.per_head_linear(o_lat, lw.w_uv)).view(t, hl * cfg.v_head_dim)
        return self.comm.all_reduce(gemm.linear(o, lw.wo))

    def _ffn(self, lw: GpuLayer, x: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        if lw.dense_gu is not None:
            return self.comm.all_reduce(self._swiglu(x, lw.dense_gu, lw.dense_down))
        logits = gemm.linear(x, lw.gate, out_f32=True)
        idx, wts = moe.route(logits, lw.gate_bias, cfg.experts_per_token, cfg.score_func, cfg.norm_topk, cfg.route_scale)
        base = self._swiglu(x, lw.shared_gu, lw.shared_down) if lw.shared_gu is not None else None
        y = moe.experts_forward(x, idx, wts, lw.w13, lw.w2, self.w.expert_lo, cfg.swiglu_limit, base)
        return self.comm.all_reduce(y)

    @torch.no_grad()
    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        """Append ``ids`` [T] (int32, device) to the context; returns fp32 logits [T, vocab]."""
        cfg, w = self.cfg, self.w
        t = ids.numel()
        if self.length + t > self.max_context:
            raise RuntimeError("sequence exceeds max_context")
        pos = torch.arange(self.length, self.length + t, dtype=torch.int32, device=self.device)
        end = self.length + t
        h = basic.embedding(ids.to(torch.int32), w.embed, 0, cfg.vocab_size)
        delta = None
        for i, lw in enumerate(w.layers):
            x = basic.rmsnorm(h, lw.attn_norm, cfg.rms_norm_eps) if delta is None else \
                basic.add_rmsnorm(h, delta, lw.attn_norm, cfg.rms_norm_eps)
            d_attn = self._attention(lw, i, x, pos, end)
            x = basic.add_rmsnorm(h, d_attn, lw.ffn_norm, cfg.rms_norm_eps)
            delta = self._ffn(lw, x)
        x = basic.add_rmsnorm(h, delta, w.norm, cfg.rms_norm_eps)
        self.length = end
        return gemm.linear(x, w.head, out_f32=True)

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new_tokens: int, chunk: int = 2048) -> tuple[list[int], torch.Tensor]:
        self.reset()
        prompt = prompt.to(self.device, torch.int32)
        logits = None
        for s in range(0, prompt.numel(), chunk):
            logits = self.forward(prompt[s:s + chunk])[-1:]
        toks, rows = [], []
        for _ in range(max_new_tokens):
            rows.append(logits[0])
            nxt = basic.argmax(logits)
            toks.append(int(nxt.item()))
            if len(toks) == max_new_tokens:
                break
            logits = self.forward(nxt)
        return toks, torch.stack(rows)
