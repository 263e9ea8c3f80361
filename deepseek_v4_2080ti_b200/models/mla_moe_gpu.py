"""GPU runtime of the MLA + routed-expert family (DeepSeek-V4-Flash-shaped, GLM-5.2-shaped): every op on the forward
path is one of this package's sm_100a kernels.

* projections: weight-decoding tcgen05 GEMM (bf16 or FP8 block-128 weights);
* attention: absorbed MLA over a paged latent cache (``ops/mla.py``): per-head absorption GEMMs run as one grouped
  GEMM, the lightning indexer scores every cached key and a radix top-k picks the keys each query attends to;
* feed-forward: dense SwiGLU for the leading layers, otherwise router top-k -> device-side plan -> grouped FP4 / FP8 /
  bf16 expert GEMMs -> weighted combine on top of the shared expert (``ops/moe.py``);
* parallelism: attention heads and the dense / shared intermediate dimension are sharded over the tensor-parallel
  group, routed experts are sharded by contiguous expert range; partial outputs are summed by ``comm``;
  optionally a layer pipeline (``parallel/pp.py``): a stage holds a contiguous layer range, receives the hidden rows
  of a chunk from the previous stage and sends them on, and the last stage shares the next token;
* weights: bf16 / FP8 block-128 / FP4 as above, or GGUF block formats quantised at load (``dense_quant``,
  ``expert_format="gguf"``) and decoded inside the GEMMs - the GLM-5.2-shaped mix is Q8_0 attention projections,
  Q4_K dense / shared feed-forward, Q2_K gate/up and IQ3_XXS down experts; or the blocks of a GGUF file as they are
  (``models/mla_gguf.py`` reads a ``glm-dsa`` checkpoint into ``RawQuant`` entries).

Same math as ``MlaMoeRuntime`` (the host path) and ``reference_cpu/mla_moe_ref.py``; see ``mla_moe.py`` for the
reference citations.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterator

import torch

from ..formats import fp8 as fp8fmt
from ..formats import gguf as G
from ..ops import basic, gemm, gguf_gemm, mla, moe
from ..ops.gemm import PackedLinear
from .mla_gguf import RawQuant
from .mla_moe import MlaMoeConfig


class _NoComm:
    world, rank = 1, 0

    def all_reduce(self, t):
        return t


def _mm(x: torch.Tensor, w, out_f32: bool = False) -> torch.Tensor:
    """Projection through whichever weight container the loader produced."""
    if isinstance(w, gguf_gemm.GGUFLinear):
        return gguf_gemm.linear(x, w, out_f32=out_f32)
    return gemm.linear(x, w, out_f32=out_f32)


GLM_GGUF_MIX = {"attn": "Q8_0", "ffn": "Q4_K", "gate_up": "Q2_K", "down": "IQ3_XXS"}


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
    offload: "moe.OffloadedExperts | None" = None      # experts in host memory behind a hot cache instead of w13 / w2


class Fp8Block:
    """An FP8 E4M3 matrix with its block-128 scale grid as a checkpoint stores it (``.weight`` float8 + ``.scale``
    fp32 [ceil(N / 128), ceil(K / 128)]); sliced on 128 boundaries for the tensor-parallel shards, handed to the GEMM as
    it is (no re-quantisation).  Reference loader: src/models/deepseek_v4/loader.py:440-662."""

    def __init__(self, w: torch.Tensor, scale: torch.Tensor):
        self.w, self.scale = w, scale.float()
        assert w.dim() == 2 and self.scale.shape == ((w.shape[0] + 127) // 128, (w.shape[1] + 127) // 128), (w.shape, scale.shape)

    @property
    def shape(self):
        return self.w.shape

    def to(self, device, *_):
        return Fp8Block(self.w.to(device), self.scale.to(device))

    def __getitem__(self, idx):
        if isinstance(idx, slice):
            idx = (idx, slice(None))
        r, c = idx
        r0, r1 = r.start or 0, self.w.shape[0] if r.stop is None else r.stop
        c0, c1 = c.start or 0, self.w.shape[1] if c.stop is None else c.stop
        assert r0 % 128 == 0 and c0 % 128 == 0 and (r1 % 128 == 0 or r1 == self.w.shape[0]) and \
            (c1 % 128 == 0 or c1 == self.w.shape[1]), "FP8 block-128 matrices are cut on 128 boundaries"
        return Fp8Block(self.w[r0:r1, c0:c1], self.scale[r0 // 128:(r1 + 127) // 128, c0 // 128:(c1 + 127) // 128])

    def dequant(self) -> torch.Tensor:
        return fp8fmt.dequantize_block128(self.w, self.scale)

    @staticmethod
    def cat(parts: list["Fp8Block"]) -> "Fp8Block":
        assert all(p.w.shape[0] % 128 == 0 for p in parts[:-1])
        return Fp8Block(torch.cat([p.w for p in parts]), torch.cat([p.scale for p in parts]))


class MlaMoeGpuWeights:
    def __init__(self, cfg: MlaMoeConfig, state: Iterator[tuple[str, torch.Tensor]], device="cuda", rank: int = 0,
                 world: int = 1, dense_fp8: bool = False, layer_range: tuple[int, int] | None = None,
                 gguf_mix: dict[str, str] | None = None, routed_tp: bool | None = None, expert_cache_slots: int = 0):
        """``rank`` / ``world``: position in the tensor/expert-parallel group (of this pipeline stage);
        ``layer_range``: the layers this stage holds (embedding only with layer 0, norm + head only with the last);
        ``gguf_mix``: GGUF types per weight class {"attn", "ffn", "gate_up", "down"} - quantised at load;
        ``routed_tp``: instead of a contiguous range of whole experts, every rank holds ALL routed experts with the
        intermediate dimension cut ``world`` ways (gate/up rows, down columns) - the reference's ``GLM_ROUTED_TP=1``
        option (src/models/glm_dsa/spec.py:282-325): no load imbalance between ranks at small batches, the same
        sum over ranks afterwards.  Default: the environment variable of the same name."""
        import os
        # > 0: the routed experts of every layer stay in pinned host memory and only this many occupy device slots
        # (ops.moe.OffloadedExperts); bf16, FP4 and GGUF experts
        self.expert_cache_slots = int(expert_cache_slots)
        self.routed_tp = (os.environ.get("GLM_ROUTED_TP", "0") == "1") if routed_tp is None else bool(routed_tp)
        if world == 1:
            self.routed_tp = False
        self.cfg, self.device, self.rank, self.world, self.dense_fp8 = cfg, torch.device(device), rank, world, dense_fp8
        self.gguf_mix = gguf_mix
        self.layer_lo, self.layer_hi = layer_range or (0, cfg.num_layers)
        assert cfg.num_heads % world == 0 and cfg.num_experts % world == 0
        self.h_local = cfg.num_heads // world
        per = cfg.num_experts // world
        self.expert_lo, self.expert_hi = rank * per, (rank + 1) * per
        if self.routed_tp:
            assert cfg.expert_intermediate % (world * 32) == 0, "routed-TP cuts the expert width into 32-aligned shards"
            self.expert_lo, self.expert_hi = 0, cfg.num_experts
        sd: dict[str, torch.Tensor] = {}
        for k, v in state:
            if k.startswith("layers."):
                li = int(k.split(".")[1])
                if not (self.layer_lo <= li < self.layer_hi):
                    continue
            if ".experts." in k:
                e = int(k.split(".experts.")[1].split(".")[0])
                if not (self.expert_lo <= e < self.expert_hi):
                    continue
            sd[k] = v
        # FP8 matrices of a checkpoint travel with their scale grids
        for k in [k for k, v in sd.items() if isinstance(v, torch.Tensor) and v.dtype == torch.float8_e4m3fn]:
            sk = k[:-len("weight")] + "scale"
            if sk not in sd:
                raise KeyError(f"{k} is FP8 but the checkpoint has no {sk}")
            sd[k] = Fp8Block(sd[k], sd.pop(sk))
        dev = self.device
        self.embed = sd["embed.weight"].to(dev, torch.bfloat16).contiguous() if self.layer_lo == 0 else None
        last = self.layer_hi == cfg.num_layers
        self.norm = sd["norm.weight"].to(dev, torch.bfloat16) if last else None
        self.head = self._lin(sd["head.weight"], "ffn") if last else None
        self.layers = [self._layer(sd, f"layers.{i}.", i < cfg.first_dense_layers)
                       if self.layer_lo <= i < self.layer_hi else None for i in range(cfg.num_layers)]
        # multi-token-prediction blocks live with the head: e_proj(norm(embed)) + h_proj(norm(hidden)) -> block -> head
        self.mtp = []
        if last and cfg.mtp_layers > 0 and "mtp.0.e_proj.weight" in sd:
            b16 = lambda t: t.to(dev, torch.bfloat16).contiguous()
            for j in range(cfg.mtp_layers):
                p = f"mtp.{j}."
                self.mtp.append({"e_proj": self._lin(sd[p + "e_proj.weight"], "ffn"), "h_proj": self._lin(sd[p + "h_proj.weight"], "ffn"),
                                 "enorm": b16(sd[p + "enorm.weight"]), "hnorm": b16(sd[p + "hnorm.weight"]),
                                 "block": self._layer(sd, p, False)})
            if self.embed is None:
                self.embed = sd["embed.weight"].to(dev, torch.bfloat16).contiguous()

    def _lin(self, w, kind: str = "ffn"):
        """A matrix of this rank as a GEMM operand.  ``RawQuant`` rows (a GGUF file's own blocks) go to the
        in-register-decode GEMM untouched; tensors are quantised per ``gguf_mix`` / ``dense_fp8`` or kept bf16."""
        if isinstance(w, RawQuant):
            if w.k % 64 == 0 and w.t in gguf_gemm.WF:
                return gguf_gemm.GGUFLinear.from_raw(w.raw.contiguous(), w.t, w.n, w.k, self.device)
            return PackedLinear.from_bf16(w.to(self.device).dequant().to(torch.bfloat16))
        if isinstance(w, Fp8Block):
            w = w.to(self.device)
            if w.shape[0] % 128 == 0 and w.shape[1] % 128 == 0:
                return PackedLinear.from_fp8(w.w.contiguous(), w.scale.contiguous())
            return PackedLinear.from_bf16(w.dequant().to(torch.bfloat16))
        w = w.to(self.device)
        if self.gguf_mix is not None:
            t = G.GGMLType[self.gguf_mix[kind]]
            if w.shape[1] % G.BLOCK_ELEMS[t] or w.shape[1] % 64:
                t = G.GGMLType.Q8_0
            if w.shape[1] % 64 == 0:
                return gguf_gemm.GGUFLinear.from_raw(G.quantize(w.float(), t), t, w.shape[0], w.shape[1], self.device)
            return PackedLinear.from_bf16(w)
        if self.dense_fp8 and w.shape[0] % 128 == 0 and w.shape[1] % 128 == 0:
            q, s = fp8fmt.quantize_block128(w.float())
            return PackedLinear.from_fp8(q, s)
        return PackedLinear.from_bf16(w)

    def _rows(self, w: torch.Tensor, group: int = 1) -> torch.Tensor:
        """Output-feature shard of a column-parallel matrix (``group`` rows stay together)."""
        n = w.shape[0] // self.world
        assert n * self.world == w.shape[0] and n % group == 0
        if isinstance(w, RawQuant):
            return w.rows(self.rank * n, (self.rank + 1) * n)
        return w[self.rank * n:(self.rank + 1) * n]

    def _cat_rows(self, parts: list):
        """Row-wise concatenation of two projections that share their input (gate | up)."""
        if isinstance(parts[0], Fp8Block):
            return Fp8Block.cat(parts)
        if isinstance(parts[0], RawQuant):
            joined = RawQuant.cat(parts)
            if joined is not None:
                return joined
            return torch.cat([p.to(self.device).dequant() for p in parts]).to(torch.bfloat16)
        return torch.cat(parts)

    def _cols(self, w: torch.Tensor) -> torch.Tensor:
        k = w.shape[1] // self.world
        return w[:, self.rank * k:(self.rank + 1) * k]

    def _lin_cols(self, w: torch.Tensor, kind: str):
        """Input-dimension (row-parallel) shard of a matrix.  GGUF blocks run along the input dimension, so the full
        matrix is quantised as a checkpoint would hold it and this rank takes its run of blocks; when the shard does
        not hold whole blocks its dequantised values are re-encoded as Q8_0 (32-wide blocks)."""
        if isinstance(w, Fp8Block):
            return self._lin(self._cols(w), kind)
        if isinstance(w, RawQuant):
            if self.world == 1:
                return self._lin(w, kind)
            kl = w.k // self.world
            part = w.cols(self.rank * kl, (self.rank + 1) * kl)
            if part is not None and kl % 64 == 0:
                return self._lin(part, kind)
            deq = w.to(self.device).dequant()[:, self.rank * kl:(self.rank + 1) * kl].contiguous()
            if kl % 64:
                return PackedLinear.from_bf16(deq.to(torch.bfloat16))
            return gguf_gemm.GGUFLinear.from_raw(G.quantize(deq, G.GGMLType.Q8_0), G.GGMLType.Q8_0, w.n, kl, self.device)
        if self.gguf_mix is None or self.world == 1:
            return self._lin(self._cols(w), kind)
        w = w.to(self.device)
        n, k = w.shape
        kl = k // self.world
        t = G.GGMLType[self.gguf_mix[kind]]
        if k % G.BLOCK_ELEMS[t] or k % 64:
            t = G.GGMLType.Q8_0
        if k % 64:
            return self._lin(self._cols(w), kind)
        raw = G.quantize(w.float(), t)
        be, bb = G.BLOCK_ELEMS[t], G.BLOCK_BYTES[t]
        if kl % be == 0 and kl % 64 == 0:
            part = raw.view(n, k // be, bb)[:, self.rank * kl // be:(self.rank + 1) * kl // be].reshape(n, -1).contiguous()
            return gguf_gemm.GGUFLinear.from_raw(part, t, n, kl, self.device)
        deq = G.dequantize(raw, t, k)[:, self.rank * kl:(self.rank + 1) * kl].contiguous()
        if kl % 64:
            return PackedLinear.from_bf16(deq.to(torch.bfloat16))
        return gguf_gemm.GGUFLinear.from_raw(G.quantize(deq, G.GGMLType.Q8_0), G.GGMLType.Q8_0, n, kl, self.device)

    def _layer(self, sd, p: str, dense: bool) -> GpuLayer:
        cfg, dev = self.cfg, self.device
        b = lambda t: t.to(dev, torch.bfloat16).contiguous()
        a = p + "attn."
        hq = cfg.qk_head_dim
        wkv_b = self._rows(sd[a + "wkv_b.weight"], cfg.qk_nope_dim + cfg.v_head_dim)
        wkv_b = (wkv_b.to(dev).dequant() if isinstance(wkv_b, Fp8Block) else wkv_b).to(dev, torch.bfloat16)
        wkv_b = wkv_b.view(self.h_local, cfg.qk_nope_dim + cfg.v_head_dim, cfg.kv_lora_rank)
        w_uk = wkv_b[:, :cfg.qk_nope_dim]                       # [H, N, C]
        lw = GpuLayer(
            attn_norm=b(sd[p + "attn_norm.weight"]), ffn_norm=b(sd[p + "ffn_norm.weight"]),
            wq_a=self._lin(sd[a + "wq_a.weight"], "attn") if cfg.q_lora_rank > 0 else None,
            q_norm=b(sd[a + "q_norm.weight"]) if cfg.q_lora_rank > 0 else None,
            wq_b=self._lin(self._rows(sd[a + ("wq_b.weight" if cfg.q_lora_rank > 0 else "wq.weight")], hq), "attn"),
            wkv_a=self._lin(sd[a + "wkv_a.weight"], "attn"), kv_norm=b(sd[a + "kv_norm.weight"]),
            w_uk_t=w_uk.transpose(1, 2).reshape(self.h_local * cfg.kv_lora_rank, cfg.qk_nope_dim).contiguous(),
            w_uv=wkv_b[:, cfg.qk_nope_dim:].reshape(self.h_local * cfg.v_head_dim, cfg.kv_lora_rank).contiguous(),
            wo=self._lin_cols(sd[a + "wo.weight"], "attn"))
        if cfg.index_heads > 0:
            # the indexer is small and replicated: every rank scores with all index heads
            lw.idx_wq, lw.idx_wk = self._lin(sd[a + "indexer.wq_b.weight"]), self._lin(sd[a + "indexer.wk.weight"])
            lw.idx_knorm, lw.idx_wproj = b(sd[a + "indexer.k_norm.weight"]), self._lin(sd[a + "indexer.weights_proj.weight"])
        f = p + "ffn."
        if dense:
            lw.dense_gu = self._lin(self._cat_rows([self._rows(sd[f + "w1.weight"]), self._rows(sd[f + "w3.weight"])]))
            lw.dense_down = self._lin_cols(sd[f + "w2.weight"], "ffn")
            return lw
        lw.gate = PackedLinear.from_bf16(sd[f + "gate.weight"].to(dev))
        lw.gate_bias = sd[f + "gate.bias"].to(dev, torch.float32)
        if cfg.num_shared_experts:
            lw.shared_gu = self._lin(self._cat_rows([self._rows(sd[f + "shared_experts.w1.weight"]),
                                                     self._rows(sd[f + "shared_experts.w3.weight"])]))
            lw.shared_down = self._lin_cols(sd[f + "shared_experts.w2.weight"], "ffn")
        es = range(self.expert_lo, self.expert_hi)
        # routed-TP: this rank's slice [r0, r1) of every expert's intermediate dimension (else the whole width)
        inter = cfg.expert_intermediate
        il = inter // self.world if self.routed_tp else inter
        r0, r1 = (self.rank * il, (self.rank + 1) * il) if self.routed_tp else (0, inter)

        def rows13(w):                       # gate / up: [I, ...] -> [il, ...]
            if not self.routed_tp:
                return w
            return w.rows(r0, r1) if isinstance(w, RawQuant) else w[r0:r1]

        def cols2(w, div: int = 1):          # down: [H, I / div] -> [H, il / div]  (div: elements per stored column)
            return w[:, r0 // div:r1 // div] if self.routed_tp else w

        first = sd[f + f"experts.{self.expert_lo}.w1.weight"]
        if isinstance(first, RawQuant):
            # a GGUF file's expert blocks as they are; gate and up stack row-wise when they share a type
            up = sd[f + f"experts.{self.expert_lo}.w3.weight"]
            if up.t == first.t and first.k % 64 == 0 and first.t in gguf_gemm.WF:
                raws = [torch.cat([rows13(sd[f + f"experts.{e}.w1.weight"]).raw, rows13(sd[f + f"experts.{e}.w3.weight"]).raw]).to(dev)
                        for e in es]
                lw.w13 = moe.ExpertWeights.from_gguf(raws, first.t, 2 * il, cfg.hidden_size)
            else:
                deq = [torch.cat([rows13(sd[f + f"experts.{e}.w1.weight"]).to(dev).dequant(),
                                  rows13(sd[f + f"experts.{e}.w3.weight"]).to(dev).dequant()]) for e in es]
                lw.w13 = moe.ExpertWeights.from_gguf([G.quantize(x, G.GGMLType.Q8_0) for x in deq], G.GGMLType.Q8_0,
                                                     2 * il, cfg.hidden_size)
            dn = sd[f + f"experts.{self.expert_lo}.w2.weight"]
            cut = (lambda w: w.cols(r0, r1)) if self.routed_tp else (lambda w: w)
            if il % 64 == 0 and dn.t in gguf_gemm.WF and cut(dn) is not None:
                lw.w2 = moe.ExpertWeights.from_gguf([cut(sd[f + f"experts.{e}.w2.weight"]).raw.to(dev) for e in es], dn.t,
                                                    cfg.hidden_size, il)
            elif il % 64 == 0:
                # the cut would split a block: this rank's columns are re-encoded as Q8_0 (32-wide blocks)
                deq = [cols2(sd[f + f"experts.{e}.w2.weight"].to(dev).dequant()).contiguous() for e in es]
                lw.w2 = moe.ExpertWeights.from_gguf([G.quantize(x, G.GGMLType.Q8_0) for x in deq], G.GGMLType.Q8_0,
                                                    cfg.hidden_size, il)
            else:
                lw.w2 = moe.ExpertWeights.from_bf16([cols2(sd[f + f"experts.{e}.w2.weight"].to(dev).dequant()).to(torch.bfloat16).contiguous()
                                                     for e in es])
        elif self.gguf_mix is not None:
            t13, t2 = G.GGMLType[self.gguf_mix["gate_up"]], G.GGMLType[self.gguf_mix["down"]]
            if il % G.BLOCK_ELEMS[t2]:
                t2 = G.GGMLType.Q8_0
            full = lambda e, n: self._expert_f32(sd, f + f"experts.{e}.{n}")
            lw.w13 = moe.ExpertWeights.from_gguf([G.quantize(torch.cat([rows13(full(e, "w1")), rows13(full(e, "w3"))]), t13)
                                                  for e in es], t13, 2 * il, cfg.hidden_size)
            lw.w2 = moe.ExpertWeights.from_gguf([G.quantize(cols2(full(e, "w2")).contiguous(), t2) for e in es], t2,
                                                cfg.hidden_size, il)
        elif cfg.expert_format == "fp4":
            cat13 = lambda e, suf: torch.cat([rows13(sd[f + f"experts.{e}.w1.{suf}"]), rows13(sd[f + f"experts.{e}.w3.{suf}"])]).to(dev)
            lw.w13 = moe.ExpertWeights.from_fp4([cat13(e, "weight") for e in es], [cat13(e, "scale") for e in es])
            # two codes per byte, one scale per 32 inputs
            lw.w2 = moe.ExpertWeights.from_fp4([cols2(sd[f + f"experts.{e}.w2.weight"], 2).contiguous().to(dev) for e in es],
                                               [cols2(sd[f + f"experts.{e}.w2.scale"], 32).contiguous().to(dev) for e in es])
        else:
            lw.w13 = moe.ExpertWeights.from_bf16([torch.cat([rows13(sd[f + f"experts.{e}.w1.weight"]),
                                                             rows13(sd[f + f"experts.{e}.w3.weight"])]).to(dev) for e in es])
            lw.w2 = moe.ExpertWeights.from_bf16([cols2(sd[f + f"experts.{e}.w2.weight"]).contiguous().to(dev) for e in es])
        if self.expert_cache_slots > 0:
            lw.offload = moe.OffloadedExperts(lw.w13, lw.w2, self.expert_cache_slots, dev, self.expert_lo)
            lw.w13 = lw.w2 = None
        return lw


    def _expert_f32(self, sd, base: str) -> torch.Tensor:
        """An expert matrix as fp32 on the device, whatever the checkpoint stores (bf16, or FP4 codes + scales)."""
        from ..formats import fp4 as fp4fmt
        w = sd[base + ".weight"].to(self.device)
        if self.cfg.expert_format == "fp4":
            return fp4fmt.dequantize(w, sd[base + ".scale"].to(self.device)).float()
        return w.float()


class MlaMoeGpuRuntime:
    """One sequence at a time (prefill in one or more chunks, then token-by-token decode) over a paged latent cache."""

    def __init__(self, cfg: MlaMoeConfig, weights: MlaMoeGpuWeights, max_context: int = 4096, block_size: int = 64, comm=None,
                 pipeline=None):
        """``comm``: communicator of this stage's tensor/expert-parallel group; ``pipeline``: a
        ``parallel.pp.PipelineLink`` when the layers are cut into stages (weights loaded with the matching
        ``layer_range``)."""
        self.cfg, self.w, self.device = cfg, weights, weights.device
        self.comm = comm or _NoComm()
        self.pp = pipeline
        self.bs = block_size
        self.max_context = max_context
        nblk = (max_context + block_size - 1) // block_size
        rows = nblk * block_size
        n = cfg.num_layers + len(weights.mtp)
        d = cfg.kv_lora_rank + cfg.qk_rope_dim
        self.mtp_length = 0
        self.spec_stats = {"steps": 0, "drafted": 0, "accepted": 0}
        self.cache = torch.zeros(n, rows, d, dtype=torch.bfloat16, device=self.device)
        self.idx_cache = torch.zeros(n, rows, max(1, cfg.index_dim), dtype=torch.bfloat16, device=self.device)
        # identity page table: block b of the sequence is physical block b (one resident sequence)
        self.block_table = torch.arange(nblk, dtype=torch.int32, device=self.device).view(1, nblk).contiguous()
        self.length = 0
        self._graphs: dict[tuple, dict] = {}
        self.launches = 0

    def reset(self) -> None:
        self.length = 0
        self.mtp_length = 0

    def _swiglu(self, x, gu, down):
        return _mm(basic.silu_mul(_mm(x, gu)), down)

    def _attention(self, lw: GpuLayer, i: int, x: torch.Tensor, pos: torch.Tensor, end: int, ld: int | None = None,
                   sparse: bool | None = None, rows: torch.Tensor | None = None, seq: torch.Tensor | None = None,
                   table: torch.Tensor | None = None) -> torch.Tensor:
        """``end``: context length after these tokens; ``ld`` / ``sparse`` override the indexer's score width and the
        dense-or-selected decision (a captured decode step fixes both for a whole context bucket).  Several sequences
        in one call: ``rows`` = physical cache row of every token, ``seq`` = its row of the page table ``table``."""
        cfg = self.cfg
        rows = pos if rows is None else rows
        table = self.block_table if table is None else table
        ld = end if ld is None else ld
        sparse = end > cfg.index_topk if sparse is None else sparse
        t = x.shape[0]
        hl = self.w.h_local
        eps = cfg.rms_norm_eps
        qin = basic.rmsnorm(_mm(x, lw.wq_a), lw.q_norm, eps) if lw.wq_a is not None else x
        q = _mm(qin, lw.wq_b)
        kv = _mm(x, lw.wkv_a)
        kidx = _mm(x, lw.idx_wk) if lw.idx_wk is not None else None
        mla.kv_append(kv, lw.kv_norm, eps, pos, rows, cfg.rope_theta, self.cache[i], cfg.kv_lora_rank, cfg.qk_rope_dim,
                      kidx, lw.idx_knorm, self.idx_cache[i] if kidx is not None else None)
        qn_t, q_pe = mla.q_prepare(q, pos, cfg.rope_theta, hl, cfg.qk_nope_dim, cfg.qk_rope_dim)
        q_lat = mla.per_head_linear(qn_t, lw.w_uk_t)
        sel = None
        if lw.idx_wq is not None and sparse:
            qi = _mm(qin, lw.idx_wq).view(t, cfg.index_heads, cfg.index_dim)
            hw = (_mm(x, lw.idx_wproj, out_f32=True) * cfg.index_heads ** -0.5).contiguous()
            world = getattr(self.comm, "world", 1)
            if world > 1 and t >= 8 * world and hasattr(self.comm, "all_gather"):
                # the indexer weights are replicated, so its work is split by query rows: every rank scores and
                # selects for a slice of the chunk and the selections (int32 [T, top-k]) are gathered
                per = (t + world - 1) // world
                lo = min(t, self.comm.rank * per)
                hi = min(t, lo + per)
                part = torch.full((per, cfg.index_topk), -1, dtype=torch.int32, device=self.device)
                if hi > lo:
                    sc = mla.indexer_scores(qi[lo:hi].contiguous(), hw[lo:hi].contiguous(), self.idx_cache[i], table,
                                            self.bs, pos[lo:hi].contiguous(), ld, cfg.index_dim ** -0.5,
                                            None if seq is None else seq[lo:hi].contiguous())
                    part[:hi - lo] = mla.topk_rows(sc, (pos[lo:hi] + 1).to(torch.int32), cfg.index_topk)
                sel = self.comm.all_gather(part).reshape(world * per, cfg.index_topk)[:t].contiguous()
            else:
                scores = mla.indexer_scores(qi, hw, self.idx_cache[i], table, self.bs, pos, ld, cfg.index_dim ** -0.5, seq)
                sel = mla.topk_rows(scores, (pos + 1).to(torch.int32), cfg.index_topk)
        o_lat = mla.attention(q_lat, q_pe, self.cache[i], table, self.bs, pos, cfg.kv_lora_rank, cfg.qk_rope_dim,
                              cfg.qk_head_dim ** -0.5, sel, seq_of_token=seq, max_keys=ld)
        o = mla.transpose_heads(mla.per_head_linear(o_lat, lw.w_uv)).view(t, hl * cfg.v_head_dim)
        return self.comm.all_reduce(_mm(o, lw.wo))

    def _ffn(self, lw: GpuLayer, x: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        if lw.dense_gu is not None:
            return self.comm.all_reduce(self._swiglu(x, lw.dense_gu, lw.dense_down))
        logits = _mm(x, lw.gate, out_f32=True)
        idx, wts = moe.route(logits, lw.gate_bias, cfg.experts_per_token, cfg.score_func, cfg.norm_topk, cfg.route_scale)
        base = self._swiglu(x, lw.shared_gu, lw.shared_down) if lw.shared_gu is not None else None
        if lw.offload is not None:
            return self.comm.all_reduce(lw.offload.forward(x, idx, wts, cfg.swiglu_limit, base))
        if getattr(self.comm, "world", 1) > 1 and hasattr(self.comm, "moe_combine"):
            # weighted combine + sum over the expert-parallel ranks in one peer-memory kernel
            return moe.experts_forward(x, idx, wts, lw.w13, lw.w2, self.w.expert_lo, cfg.swiglu_limit, base, comm=self.comm)
        y = moe.experts_forward(x, idx, wts, lw.w13, lw.w2, self.w.expert_lo, cfg.swiglu_limit, base)
        return self.comm.all_reduce(y)

    @torch.no_grad()
    def mtp_draft(self, hidden: torch.Tensor, next_ids: torch.Tensor, depth: int = 0) -> torch.Tensor:
        """Multi-token-prediction block ``depth`` over positions [mtp_length, mtp_length + T): ``hidden`` [T, H] are
        the main model's final residual rows at those positions, ``next_ids`` [T] the tokens that follow them.
        Returns fp32 logits [T, vocab] for the token after next.  (Reference: MTPBlock,
        src/models/deepseek_v4/runtime.py:4610-4642, draft_with_mtp :4904.)"""
        cfg, w = self.cfg, self.w
        m = w.mtp[depth]
        t = hidden.shape[0]
        pos = torch.arange(self.mtp_length, self.mtp_length + t, dtype=torch.int32, device=self.device)
        emb = basic.embedding(next_ids.to(torch.int32), w.embed, 0, cfg.vocab_size)
        h = _mm(basic.rmsnorm(emb, m["enorm"], cfg.rms_norm_eps), m["e_proj"])
        basic.add_(h, _mm(basic.rmsnorm(hidden, m["hnorm"], cfg.rms_norm_eps), m["h_proj"]))
        lw = m["block"]
        li = cfg.num_layers + depth
        x = basic.rmsnorm(h, lw.attn_norm, cfg.rms_norm_eps)
        d_attn = self._attention(lw, li, x, pos, self.mtp_length + t)
        x = basic.add_rmsnorm(h, d_attn, lw.ffn_norm, cfg.rms_norm_eps)
        delta = self._ffn(lw, x)
        x = basic.add_rmsnorm(h, delta, w.norm, cfg.rms_norm_eps)
        self.mtp_length += t
        return _mm(x, w.head, out_f32=True)

    @torch.no_grad()
    def generate_mtp(self, prompt: torch.Tensor, max_new_tokens: int, chunk: int = 2048, draft_override=None) -> list[int]:
        """Greedy generation with depth-1 speculative drafting: each step verifies [token, draft] in one two-row
        pass; an accepted draft yields two tokens per pass, a rejected one rolls the latent cache back by a row.
        The stream equals plain greedy decoding.  ``draft_override(n_emitted) -> int | None`` replaces the draft
        (tests use it to force acceptance)."""
        assert self.pp is None and self.w.mtp, "speculative decoding needs the MTP block and an unsplit model"
        self.reset()
        self.spec_stats = {"steps": 0, "drafted": 0, "accepted": 0}
        prompt = prompt.to(self.device, torch.int32)
        hid, logits = [], None
        for s in range(0, prompt.numel(), chunk):
            logits, h = self.forward(prompt[s:s + chunk], return_hidden=True)
            hid.append(h)
        tok = basic.argmax(logits[-1:])
        out = [int(tok.item())]
        d_logits = self.mtp_draft(torch.cat(hid), torch.cat([prompt[1:], tok.to(torch.int32)]))
        draft = basic.argmax(d_logits[-1:])
        while len(out) < max_new_tokens:
            if draft_override is not None:
                forced = draft_override(len(out))
                if forced is not None:
                    draft = torch.tensor([forced], dtype=torch.int32, device=self.device)
            pair = torch.cat([tok.to(torch.int32), draft.to(torch.int32)])
            logits, h = self.forward(pair, return_hidden=True)
            nxt = basic.argmax(logits)                      # [2]: token after `tok`, token after `draft`
            self.spec_stats["steps"] += 1
            self.spec_stats["drafted"] += 1
            ok = bool((nxt[0] == draft[0]).item())
            if ok:
                self.spec_stats["accepted"] += 1
                out.append(int(nxt[0].item()))
                if len(out) < max_new_tokens:
                    out.append(int(nxt[1].item()))
                tok = nxt[1:2]
                d_logits = self.mtp_draft(h, nxt.to(torch.int32))
            else:
                self.length -= 1                            # the draft's cache row is overwritten by the next pass
                out.append(int(nxt[0].item()))
                tok = nxt[0:1]
                d_logits = self.mtp_draft(h[:1], nxt[:1].to(torch.int32))
            draft = basic.argmax(d_logits[-1:])
        return out[:max_new_tokens]

    @torch.no_grad()
    def forward(self, ids: torch.Tensor, return_hidden: bool = False):
        """Append ``ids`` [T] (int32, device) to the context; returns fp32 logits [T, vocab] (on the last pipeline
        stage; earlier stages send their hidden rows on and return None)."""
        cfg, w = self.cfg, self.w
        t = ids.numel()
        if self.length + t > self.max_context:
            raise RuntimeError("sequence exceeds max_context")
        pos = torch.arange(self.length, self.length + t, dtype=torch.int32, device=self.device)
        end = self.length + t
        if w.layer_lo == 0:
            h = basic.embedding(ids.to(torch.int32), w.embed, 0, cfg.vocab_size)
        else:
            h = self.pp.recv_hidden(t, cfg.hidden_size)
        delta = None
        for i, lw in enumerate(w.layers):
            if lw is None:
                continue
            x = basic.rmsnorm(h, lw.attn_norm, cfg.rms_norm_eps) if delta is None else \
                basic.add_rmsnorm(h, delta, lw.attn_norm, cfg.rms_norm_eps)
            d_attn = self._attention(lw, i, x, pos, end)
            x = basic.add_rmsnorm(h, d_attn, lw.ffn_norm, cfg.rms_norm_eps)
            delta = self._ffn(lw, x)
        self.length = end
        self.launches = 0
        if w.layer_hi < cfg.num_layers:
            basic.add_(h, delta)
            self.pp.send_hidden(h)
            return None
        x = basic.add_rmsnorm(h, delta, w.norm, cfg.rms_norm_eps)          # h becomes the final residual stream
        logits = _mm(x, w.head, out_f32=True)
        return (logits, h) if return_hidden else logits

    def _decode_body(self, ent: dict, ld: int, sparse: bool) -> torch.Tensor:
        """One token through every layer with device-side position (static buffers: capturable)."""
        cfg, w = self.cfg, self.w
        pos = ent["pos"]
        h = basic.embedding(ent["ids"], w.embed, 0, cfg.vocab_size)
        delta = None
        for i, lw in enumerate(w.layers):
            x = basic.rmsnorm(h, lw.attn_norm, cfg.rms_norm_eps) if delta is None else \
                basic.add_rmsnorm(h, delta, lw.attn_norm, cfg.rms_norm_eps)
            d_attn = self._attention(lw, i, x, pos, ld, ld, sparse)
            x = basic.add_rmsnorm(h, d_attn, lw.ffn_norm, cfg.rms_norm_eps)
            delta = self._ffn(lw, x)
        x = basic.add_rmsnorm(h, delta, w.norm, cfg.rms_norm_eps)
        ent["logits"] = _mm(x, w.head, out_f32=True)
        return basic.argmax(ent["logits"])

    @torch.no_grad()
    def decode_step(self, token: torch.Tensor, use_graph: bool = True) -> torch.Tensor:
        """Append one token (int32 [1], device) and return the greedy next token [1].  The step is captured once per
        context bucket (power of two; the indexer scores that many positions and masks by the device-side position)
        and replayed: one graph launch instead of a few dozen kernel launches per layer.  Not for pipeline stages."""
        assert self.pp is None and self.w.layer_lo == 0 and self.w.layer_hi == self.cfg.num_layers
        end = self.length + 1
        if end > self.max_context:
            raise RuntimeError("sequence exceeds max_context")
        rows = self.cache.shape[1]
        ld = min(rows, 1 << max(10, (end - 1).bit_length()))
        sparse = end > self.cfg.index_topk
        key = (ld, sparse)
        ent = self._graphs.get(key)
        if ent is None:
            ent = {"ids": torch.zeros(1, dtype=torch.int32, device=self.device),
                   "pos": torch.zeros(1, dtype=torch.int32, device=self.device), "graph": None, "out": None}
            self._graphs[key] = ent
        ent["ids"].copy_(token.reshape(1))
        ent["pos"].fill_(self.length)
        if not use_graph:
            out = self._decode_body(ent, ld, sparse)
        else:
            if ent["graph"] is None:
                self._decode_body(ent, ld, sparse)      # warm-up outside capture; rewrites the same cache row later
                torch.cuda.synchronize()
                from ..ops import _lib
                l0 = _lib.LAUNCHES
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    ent["out"] = self._decode_body(ent, ld, sparse)
                ent["graph"], ent["launches"] = g, _lib.LAUNCHES - l0
            ent["graph"].replay()
            out = ent["out"]
            self.launches = ent["launches"]
        self.last_logits = ent["logits"]
        self.length = end
        return out

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new_tokens: int, chunk: int = 2048) -> tuple[list[int], torch.Tensor]:
        self.reset()
        prompt = prompt.to(self.device, torch.int32)
        last_stage = self.w.layer_hi == self.cfg.num_layers
        logits = None
        for s in range(0, prompt.numel(), chunk):       # stages overlap: a stage starts chunk c + 1 once c is sent on
            out = self.forward(prompt[s:s + chunk])
            logits = out[-1:] if out is not None else None
        toks, rows = [], []
        graph = self.pp is None and self.w.layer_lo == 0 and last_stage
        for _ in range(max_new_tokens):
            nxt = basic.argmax(logits) if last_stage else None
            if last_stage:
                rows.append(logits[0].clone())
            if self.pp is not None:
                nxt = self.pp.share_token(nxt)
            toks.append(int(nxt.item()))
            if len(toks) == max_new_tokens:
                break
            if graph:
                self.decode_step(nxt.to(torch.int32))
                logits = self.last_logits
            else:
                logits = self.forward(nxt)
        if self.pp is not None:
            self.pp.drain()
        return toks, (torch.stack(rows) if rows else torch.empty(0))


class MlaMoeBatchRuntime(MlaMoeGpuRuntime):
    """Several sequences over ONE paged latent cache: ``max_slots`` page-table rows, pages handed out from a free list
    as sequences grow and returned by ``free``; ``prefill`` appends a chunk to one sequence, ``decode`` advances any
    subset of the sequences by one token each in a single pass (the GEMMs, the router and the experts see B rows; the
    indexer, the top-k and the sparse attention address each row's own pages through ``seq_of_token``).
    Reference behaviour: the batched decode / verify of the resident engine
    (cpp_engine/include/persistent_engine.hpp:24-208), config rows "batch 64" (DSV4-Flash) and "batch 16" (GLM)."""
    single_sequence = False
    exposes_logits = True        # ``last_logits`` [rows, vocab] fp32 after prefill (last row) and decode (one row per slot)

    def __init__(self, cfg: MlaMoeConfig, weights: MlaMoeGpuWeights, max_slots: int = 4, max_context: int = 4096,
                 block_size: int = 64, num_blocks: int | None = None, comm=None):
        self.max_slots = int(max_slots)
        per_seq = (max_context + block_size - 1) // block_size
        self.num_blocks = int(num_blocks) if num_blocks else per_seq * self.max_slots
        # the parent sizes the caches from max_context: give it the pool's capacity, then restore the per-sequence limit
        super().__init__(cfg, weights, max_context=self.num_blocks * block_size, block_size=block_size, comm=comm)
        assert self.pp is None and weights.layer_lo == 0 and weights.layer_hi == cfg.num_layers, "no pipeline stages here"
        self.max_context = max_context
        self.blocks_per_seq = per_seq
        self.last_logits = torch.zeros(1, cfg.vocab_size, dtype=torch.float32, device=self.device)
        self.table = torch.zeros(self.max_slots, per_seq, dtype=torch.int32, device=self.device)
        self._table_host = [[-1] * per_seq for _ in range(self.max_slots)]
        self._free_pages = list(range(self.num_blocks - 1, -1, -1))
        self._free_slots = list(range(self.max_slots - 1, -1, -1))
        self.lengths = [0] * self.max_slots

    # ---- slots and pages
    def allocate(self) -> int:
        if not self._free_slots:
            raise RuntimeError("no free slot")
        s = self._free_slots.pop()
        self.lengths[s] = 0
        return s

    def free(self, slot: int) -> None:
        for b, page in enumerate(self._table_host[slot]):
            if page >= 0:
                self._free_pages.append(page)
                self._table_host[slot][b] = -1
        self.lengths[slot] = 0
        self._free_slots.append(slot)

    def free_pages(self) -> int:
        return len(self._free_pages)

    def _ensure_pages(self, slot: int, end: int) -> None:
        if end > self.max_context:
            raise RuntimeError("sequence exceeds max_context")
        need = (end + self.bs - 1) // self.bs
        row, changed = self._table_host[slot], False
        for b in range(need):
            if row[b] < 0:
                if not self._free_pages:
                    raise RuntimeError("the latent cache has no free page")
                row[b] = self._free_pages.pop()
                changed = True
        if changed:
            self.table[slot] = torch.tensor([max(p, 0) for p in row], dtype=torch.int32).to(self.device, non_blocking=False)

    def _rows_of(self, slot: int, lo: int, hi: int) -> list[int]:
        row, bs = self._table_host[slot], self.bs
        return [row[p // bs] * bs + p % bs for p in range(lo, hi)]

    # ---- passes
    def _run(self, ids: torch.Tensor, pos_l: list[int], rows_l: list[int], seq_l: list[int], end_max: int) -> torch.Tensor:
        cfg, w, dev = self.cfg, self.w, self.device
        i32 = lambda v: torch.tensor(v, dtype=torch.int32).to(dev)
        pos, rows, seq = i32(pos_l), i32(rows_l), i32(seq_l)
        # the indexer scores [0, ld) of every row's sequence and masks beyond the row's own position; rows shorter than
        # the top-k width simply select everything they can see
        ld = min(self.blocks_per_seq * self.bs, max(64, (end_max + 63) // 64 * 64))
        sparse = cfg.index_heads > 0 and end_max > cfg.index_topk
        h = basic.embedding(ids.to(torch.int32), w.embed, 0, cfg.vocab_size)
        delta = None
        for i, lw in enumerate(w.layers):
            x = basic.rmsnorm(h, lw.attn_norm, cfg.rms_norm_eps) if delta is None else \
                basic.add_rmsnorm(h, delta, lw.attn_norm, cfg.rms_norm_eps)
            d_attn = self._attention(lw, i, x, pos, end_max, ld, sparse, rows=rows, seq=seq, table=self.table)
            x = basic.add_rmsnorm(h, d_attn, lw.ffn_norm, cfg.rms_norm_eps)
            delta = self._ffn(lw, x)
        x = basic.add_rmsnorm(h, delta, w.norm, cfg.rms_norm_eps)
        return x

    @torch.no_grad()
    def prefill(self, slot: int, ids: torch.Tensor, chunk: int = 2048) -> torch.Tensor:
        """Append ``ids`` to sequence ``slot``; returns the greedy next token [1]."""
        ids = ids.to(self.device, torch.int32).reshape(-1)
        x = None
        for s0 in range(0, ids.numel(), chunk):
            part = ids[s0:s0 + chunk]
            lo = self.lengths[slot]
            hi = lo + part.numel()
            self._ensure_pages(slot, hi)
            x = self._run(part, list(range(lo, hi)), self._rows_of(slot, lo, hi), [slot] * (hi - lo), hi)
            self.lengths[slot] = hi
        self.last_logits = _mm(x[-1:].contiguous(), self.w.head, out_f32=True)
        return basic.argmax(self.last_logits)

    @torch.no_grad()
    def decode(self, slots: list[int], tokens: torch.Tensor) -> torch.Tensor:
        """One token for each of ``slots`` (distinct); returns the greedy next tokens [B]."""
        assert len(set(slots)) == len(slots) and tokens.numel() == len(slots)
        pos_l, rows_l = [], []
        for s in slots:
            p = self.lengths[s]
            self._ensure_pages(s, p + 1)
            pos_l.append(p)
            rows_l += self._rows_of(s, p, p + 1)
        x = self._run(tokens.to(self.device, torch.int32).reshape(-1), pos_l, rows_l, list(slots), max(pos_l) + 1)
        for s in slots:
            self.lengths[s] += 1
        self.last_logits = _mm(x, self.w.head, out_f32=True)
        return basic.argmax(self.last_logits)

    @torch.no_grad()
    def verify(self, slot: int, tokens: torch.Tensor) -> tuple[int, int]:
        """Speculative verification on one sequence: ``tokens`` = [t0, d1, ..., dK] where t0 is the last accepted token
        (not yet in the cache) and d1..dK are drafts.  One pass scores all K + 1 rows; draft d(i+1) is accepted while
        it equals the greedy choice after row i.  The cache keeps t0 and the accepted drafts only (the latent cache
        rolls back by shortening the sequence; later rows are overwritten).  Returns (accepted drafts, next token)."""
        ids = tokens.to(self.device, torch.int32).reshape(-1)
        k1 = ids.numel()
        lo = self.lengths[slot]
        self._ensure_pages(slot, lo + k1)
        x = self._run(ids, list(range(lo, lo + k1)), self._rows_of(slot, lo, lo + k1), [slot] * k1, lo + k1)
        self.last_logits = _mm(x, self.w.head, out_f32=True)
        choice = basic.argmax(self.last_logits).tolist()
        drafts = ids[1:].tolist()
        accepted = 0
        while accepted < len(drafts) and drafts[accepted] == choice[accepted]:
            accepted += 1
        self.lengths[slot] = lo + 1 + accepted
        return accepted, int(choice[accepted])
