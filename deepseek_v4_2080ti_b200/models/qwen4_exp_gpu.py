"""GPU runtime of the Qwen4-Exp-style decoder: the same model as ``models/qwen4_exp_ref.py`` (hyper-connection streams,
Gated-DeltaNet and QSA layers, routed experts, hashed n-gram injection) with the heavy operators on this package's
kernels:

* every projection: the tcgen05 GEMM (``ops.gemm.linear``, bf16 weights);
* Gated DeltaNet: depthwise convolution + SiLU (``ops.basic.conv_silu``), then the chunked tensor-core scan
  (``ops.gdn.chunked``) for a chunk of tokens or the fused step kernel for one;
* QSA layers: selection by the block-pooled indexer (tensor code on the device), attention over the selected tokens
  by the gather-based tensor-core kernel (``ops.qsa.attention``);
* routed experts: device routing plan + grouped GEMMs + weighted combine (``ops.moe.experts_forward``).

The hyper-connection mixers, norms and the n-gram injection are small element-wise / low-rank tensor code and stay
as PyTorch expressions on the device.  One sequence; ``forward(ids)`` appends to the context and returns fp32 logits.
Reference: src/models/qwen4_exp/model.py:137-421 (decoder loop), attention.py:312-436 (Gated DeltaNet), :461-737
(QSA), moe.py (router + experts), hyper_connection.py.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ..ops import basic, gdn, gemm, moe, qsa
from ..ops.gemm import PackedLinear
from . import qwen4_exp_components as C
from .qwen4_exp_ref import Qwen4ExpConfig, Qwen4ExpRef, _rms


class Qwen4ExpGpu(Qwen4ExpRef):
    def __init__(self, cfg: Qwen4ExpConfig, weights: dict[str, torch.Tensor], max_context: int = 512, device="cuda"):
        self.device = torch.device(device)
        assert cfg.head_dim == 128 and cfg.conv_kernel == 4, "the kernels are built for 128-wide heads and a 4-tap convolution"
        super().__init__(cfg, weights, max_context)
        dev = self.device
        self.w = {k: v.to(dev) for k, v in self.w.items()}
        self.cos, self.sin = self.cos.to(dev), self.sin.to(dev)
        self.lin: dict[str, PackedLinear] = {}
        self.experts: dict[int, tuple[moe.ExpertWeights, moe.ExpertWeights]] = {}
        kd = cfg.linear_k_heads * 128
        for i, lt in enumerate(cfg.layer_types):
            p = f"layers.{i}."
            if lt == "linear":
                a = p + "linear_attn."
                # q|k|v and z in one GEMM; a and b (the gate inputs) are a second, narrow one
                self._pack(a + "qkvz", torch.cat([self.w[a + "in_proj_qkv"], self.w[a + "in_proj_z"]]))
                self._pack(a + "ab", torch.cat([self.w[a + "in_proj_a"], self.w[a + "in_proj_b"]]))
                self._pack(a + "out_proj", self.w[a + "out_proj"])
                self.w[a + "conv_t"] = self.w[a + "conv1d"].to(torch.bfloat16).contiguous()
            else:
                a = p + "self_attn."
                self._pack(a + "qkv", torch.cat([self.w[a + "q_proj"], self.w[a + "k_proj"], self.w[a + "v_proj"],
                                                 self.w[a + "index_qk_proj"]]))
                self._pack(a + "o_proj", self.w[a + "o_proj"])
            m = p + "mlp."
            self._pack(m + "shared_gu", torch.cat([self.w[m + "shared.gate_proj"], self.w[m + "shared.up_proj"]]))
            self._pack(m + "shared_down", self.w[m + "shared.down_proj"])
            w13 = [torch.cat([self.w[m + f"experts.{e}.gate_proj"], self.w[m + f"experts.{e}.up_proj"]]).to(torch.bfloat16)
                   for e in range(cfg.num_experts)]
            w2 = [self.w[m + f"experts.{e}.down_proj"].to(torch.bfloat16) for e in range(cfg.num_experts)]
            self.experts[i] = (moe.ExpertWeights.from_bf16(w13), moe.ExpertWeights.from_bf16(w2))
        self._pack("lm_head", self.w["lm_head"])
        self._kd = kd
        self.reset()

    def _pack(self, name: str, w: torch.Tensor) -> None:
        n = w.shape[0]
        pad = (-n) % 16                                   # the GEMM wants feature counts in steps of 16
        if pad:
            w = torch.cat([w, torch.zeros(pad, w.shape[1], device=w.device, dtype=w.dtype)])
        self.lin[name] = PackedLinear.from_bf16(w.to(self.device))
        self.lin[name].rows = n

    def _mm(self, x: torch.Tensor, name: str, out_f32: bool = False) -> torch.Tensor:
        pl = self.lin[name]
        y = gemm.linear(x.to(torch.bfloat16).contiguous(), pl, out_f32=out_f32)
        return y[:, :pl.rows]

    def reset(self) -> None:
        cfg = self.cfg
        dev = getattr(self, "device", torch.device("cpu"))
        self.length = 0
        self.history = torch.full((1, cfg.ngram_size - 1), cfg.eos_token_id, dtype=torch.long)
        self.cache = []
        for lt in cfg.layer_types:
            if lt == "linear":
                cdim = 2 * cfg.linear_k_heads * 128 + cfg.linear_v_heads * 128
                self.cache.append({"tail": torch.zeros(cfg.conv_kernel - 1, cdim, dtype=torch.bfloat16, device=dev),
                                   "state": torch.zeros(cfg.linear_v_heads, 128, 128, dtype=torch.float32, device=dev)})
            else:
                self.cache.append({"kv": qsa.QsaCache(cfg.num_kv_heads, self.max_context, dev) if dev.type == "cuda" else None,
                                   "index_k": torch.zeros(0, cfg.indexer_head_dim, device=dev)})
        self.ple_conv = {i: torch.zeros(cfg.hc_count * cfg.hidden_size, (cfg.ple_conv_kernel - 1) * cfg.ngram_size, device=dev)
                         for i in cfg.ple_layers}

    def snapshot(self) -> dict:
        raise NotImplementedError("snapshots of the device caches are not implemented; use Qwen4ExpRef for that")

    # ---- pieces
    def _ple(self, i: int, streams: torch.Tensor, history: torch.Tensor) -> torch.Tensor:
        cfg, w, p = self.cfg, self.w, f"layers.{i}.ple."
        s, h, hc = streams.shape[0], cfg.hidden_size, cfg.hc_count
        rows = C.ngram_row_ids(history, s, cfg.ngram_size, cfg.heads_per_ngram, self._sizes, self._offsets, self._mult[i],
                               cfg.eos_token_id)[0].to(self.device)                       # hashed on the host: integer code
        emb = w[p + "table"][rows].flatten(-2)
        key = C._group_rms(F.linear(emb, w[p + "key_proj"]), w[p + "norm_key"], h, cfg.rms_norm_eps).unflatten(-1, (hc, h))
        value = F.linear(emb, w[p + "value_proj"])
        query = C._group_rms(streams, w[p + "norm_query"], h, cfg.rms_norm_eps).unflatten(-1, (hc, h))
        gate = (key * query).sum(-1, keepdim=True) / math.sqrt(h)
        gate = gate.abs().clamp_min(1e-6).sqrt() * gate.sign()
        gated = (torch.sigmoid(gate) * value.unsqueeze(-2)).flatten(-2)
        normed = C._group_rms(gated, w[p + "norm_conv"], h, cfg.rms_norm_eps)
        x = torch.cat([self.ple_conv[i], normed.t()], -1)
        self.ple_conv[i] = x[:, -self.ple_conv[i].shape[1]:].clone() if self.ple_conv[i].shape[1] else self.ple_conv[i]
        conv = F.conv1d(x[None], w[p + "conv1d"][:, None, :], None, dilation=cfg.ngram_size, groups=x.shape[0])[0]
        return gated + F.silu(conv[:, -s:]).t()

    def _deltanet(self, i: int, x: torch.Tensor) -> torch.Tensor:
        cfg, w, p, c = self.cfg, self.w, f"layers.{i}.linear_attn.", self.cache[i]
        s = x.shape[0]
        kd, vd, hv, hk = self._kd, cfg.linear_v_heads * 128, cfg.linear_v_heads, cfg.linear_k_heads
        xb = x.to(torch.bfloat16).contiguous()
        proj = self._mm(xb, p + "qkvz")                                                  # [S, 2kd + vd | vd]
        ab = self._mm(xb, p + "ab", out_f32=True)                                        # [S, hv | hv] fp32
        g = (-w[p + "A_log"].exp() * F.softplus(ab[:, :hv] + w[p + "dt_bias"])).contiguous()
        beta = torch.sigmoid(ab[:, hv:]).contiguous()
        mixed = basic.conv_silu(proj[:, :2 * kd + vd], w[p + "conv_t"], c["tail"])       # [S, 2kd + vd] bf16, tail updated
        o = gdn.chunked(mixed, 0, kd, 2 * kd, g, beta, c["state"], hv, hk)                # [S, hv, 128] bf16, state updated
        z = proj[:, 2 * kd + vd:].float().reshape(s, hv, 128)
        o = _rms(o, w[p + "norm"], cfg.rms_norm_eps) * F.silu(z)
        return self._mm(o.reshape(s, vd), p + "out_proj").float()

    def _qsa(self, i: int, x: torch.Tensor, past: int) -> torch.Tensor:
        cfg, w, p, c = self.cfg, self.w, f"layers.{i}.self_attn.", self.cache[i]
        s, d, di = x.shape[0], cfg.head_dim, cfg.indexer_head_dim
        end = past + s
        cos, sin = self.cos[:, past:end], self.sin[:, past:end]
        nq, nkv, ni = cfg.num_heads * 2 * d, cfg.num_kv_heads * d, cfg.indexer_heads * di
        proj = self._mm(x, p + "qkv", out_f32=True)                                      # q (with gates) | k | v | index q | index k
        qg, k, v, qk = proj.split([nq, nkv, nkv, ni + di], -1)
        qi = _rms(qk[:, :ni].reshape(s, -1, di), w[p + "q_layernorm"], cfg.rms_norm_eps)
        qi = C.apply_rotary_half(qi[None], cos, sin)
        c["index_k"] = torch.cat([c["index_k"], qk[:, ni:]])
        sel = C.qsa_select(qi, c["index_k"][None], w[p + "k_layernorm"], self.cos[:, :end], self.sin[:, :end], past,
                           cfg.indexer_budget, cfg.indexer_compress_ratio, cfg.rms_norm_eps)[0].contiguous()
        qg = qg.reshape(s, cfg.num_heads, 2 * d)
        q, gate = qg[..., :d], qg[..., d:].reshape(s, -1)
        q = C.apply_rotary_half(_rms(q, w[p + "q_norm"], cfg.rms_norm_eps)[None], cos, sin)[0]
        k = C.apply_rotary_half(_rms(k.reshape(s, -1, d), w[p + "k_norm"], cfg.rms_norm_eps)[None], cos, sin)[0]
        c["kv"].append(k.to(torch.bfloat16), v.reshape(s, -1, d).to(torch.bfloat16))
        pos = torch.arange(past, end, dtype=torch.int32, device=self.device)
        o = qsa.attention(q.to(torch.bfloat16).contiguous(), c["kv"], sel, pos, d ** -0.5).reshape(s, -1).float()
        return self._mm(o * torch.sigmoid(gate), p + "o_proj").float()

    def _mlp(self, i: int, x: torch.Tensor) -> torch.Tensor:
        cfg, w, p = self.cfg, self.w, f"layers.{i}.mlp."
        xb = x.to(torch.bfloat16).contiguous()
        val, idx = C.topk_softmax_router(x, w[p + "gate"], cfg.experts_per_token, cfg.norm_topk)
        w13, w2 = self.experts[i]
        routed = moe.experts_forward(xb, idx.to(torch.int32).contiguous(), val.float().contiguous(), w13, w2, 0).float()
        gu = self._mm(xb, p + "shared_gu")
        shared = self._mm(basic.silu_mul(gu.contiguous()), p + "shared_down").float()
        return routed + torch.sigmoid(F.linear(x, w[p + "shared_gate"])) * shared

    # ---- forward
    @torch.no_grad()
    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        ids_host = ids.reshape(-1).long().cpu()
        s, past = ids_host.numel(), self.length
        if past + s > self.max_context:
            raise RuntimeError("sequence exceeds max_context")
        history = torch.cat([self.history, ids_host[None]], 1)
        h, hc, eps = cfg.hidden_size, cfg.hc_count, cfg.rms_norm_eps
        streams = w["embed"][ids_host.to(self.device)].repeat(1, hc)
        for i, lt in enumerate(cfg.layer_types):
            p = f"layers.{i}."
            if i in cfg.ple_layers:
                streams = streams + self._ple(i, streams, history)
            mixed, inject = C.gated_residual(streams, w[p + "attn_hc.hc_norm"], w[p + "attn_hc.down"], w[p + "attn_hc.up"],
                                             w[p + "attn_hc.inject"], hc, h, eps)
            attn = self._deltanet(i, mixed.float()) if lt == "linear" else self._qsa(i, mixed.float(), past)
            streams = C.inject_into_streams(attn, streams, inject.float())
            mixed, inject = C.gated_residual(streams, w[p + "mlp_hc.hc_norm"], w[p + "mlp_hc.down"], w[p + "mlp_hc.up"],
                                             w[p + "mlp_hc.inject"], hc, h, eps)
            streams = C.inject_into_streams(self._mlp(i, mixed.float()), streams, inject.float())
        self.length = past + s
        self.history = history[:, -(cfg.ngram_size - 1):].clone()
        final = C.gated_residual(streams, w["final.hc_norm"], w["final.down"], w["final.up"], None, hc, h, eps)
        return self._mm(final, "lm_head", out_f32=True)
