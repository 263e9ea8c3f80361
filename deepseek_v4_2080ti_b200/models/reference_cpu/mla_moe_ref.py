"""fp32 PyTorch oracle for the MLA + MoE family: whole-sequence forward, per-head K/V expanded from
the latent (no absorption, no cache), routed experts dequantised to fp32 and applied expert by
expert.  Written after the reference's plain PyTorch paths (MLA: src/models/glm_dsa/architecture.py:345-406;
FP4 dequantisation: src/kernels/ops.py:110-155; gate and expert: src/models/deepseek_v4/runtime.py:1703-1731,
2626-2640); used only by tests."""
from __future__ import annotations

import torch

from ...formats import fp4 as fp4fmt
from ..mla_moe import MlaMoeConfig, rms_norm, rope_interleaved, route, swiglu


class MlaMoeRef:
    def __init__(self, cfg: MlaMoeConfig, state):
        self.cfg = cfg
        self.sd = {k: v for k, v in state}

    def _w(self, name: str) -> torch.Tensor:
        return self.sd[name].float()

    def _expert(self, prefix: str, n: str) -> torch.Tensor:
        w = self.sd[prefix + f"{n}.weight"]
        if self.cfg.expert_format == "fp4":
            return fp4fmt.dequantize(w, self.sd[prefix + f"{n}.scale"])
        return w.float()

    @torch.no_grad()
    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        t = ids.numel()
        pos = torch.arange(t)
        h = self._w("embed.weight")[ids.long()]
        causal = pos[None, :] <= pos[:, None]
        for i in range(cfg.num_layers):
            p = f"layers.{i}."
            a = p + "attn."
            x = rms_norm(h, self._w(p + "attn_norm.weight"), cfg.rms_norm_eps)
            if cfg.q_lora_rank > 0:
                qin = rms_norm(x @ self._w(a + "wq_a.weight").t(), self._w(a + "q_norm.weight"), cfg.rms_norm_eps)
                q = qin @ self._w(a + "wq_b.weight").t()
            else:
                qin = x
                q = x @ self._w(a + "wq.weight").t()
            q = q.view(t, cfg.num_heads, cfg.qk_head_dim)
            q = torch.cat([q[..., :cfg.qk_nope_dim], rope_interleaved(q[..., cfg.qk_nope_dim:], pos, cfg.rope_theta)], -1)
            kv = x @ self._w(a + "wkv_a.weight").t()
            c = rms_norm(kv[:, :cfg.kv_lora_rank], self._w(a + "kv_norm.weight"), cfg.rms_norm_eps)
            k_pe = rope_interleaved(kv[:, cfg.kv_lora_rank:], pos, cfg.rope_theta)
            kvb = (c @ self._w(a + "wkv_b.weight").t()).view(t, cfg.num_heads, cfg.qk_nope_dim + cfg.v_head_dim)
            k = torch.cat([kvb[..., :cfg.qk_nope_dim], k_pe[:, None, :].expand(-1, cfg.num_heads, -1)], -1)
            v = kvb[..., cfg.qk_nope_dim:]
            mask = causal
            if cfg.index_heads > 0 and t > cfg.index_topk:
                ki = rms_norm(x @ self._w(a + "indexer.wk.weight").t(), self._w(a + "indexer.k_norm.weight"), cfg.rms_norm_eps)
                qi = (qin @ self._w(a + "indexer.wq_b.weight").t()).view(t, cfg.index_heads, cfg.index_dim)
                hw = (x @ self._w(a + "indexer.weights_proj.weight").t()) * cfg.index_heads ** -0.5
                sc = (torch.einsum("thd,sd->ths", qi, ki).relu() * hw[:, :, None]).sum(1) * cfg.index_dim ** -0.5
                sc = sc.masked_fill(~causal, float("-inf"))
                # a query that sees fewer than topk keys keeps all of them (its run also had end <= topk or -inf picks)
                sel = sc.topk(cfg.index_topk, -1).indices
                keep = torch.zeros(t, t, dtype=torch.bool).scatter_(1, sel, True)
                mask = causal & keep
            s = torch.einsum("thd,shd->ths", q, k) * cfg.qk_head_dim ** -0.5
            s = s.masked_fill(~mask[:, None, :], float("-inf"))
            o = torch.einsum("ths,shv->thv", s.softmax(-1), v).reshape(t, -1)
            h = h + o @ self._w(a + "wo.weight").t()
            x = rms_norm(h, self._w(p + "ffn_norm.weight"), cfg.rms_norm_eps)
            f = p + "ffn."
            if i < cfg.first_dense_layers:
                y = swiglu(x, self._w(f + "w1.weight"), self._w(f + "w3.weight"), self._w(f + "w2.weight"))
            else:
                wts, idx = route(cfg, x, self._w(f + "gate.weight"), self.sd[f + "gate.bias"])
                y = torch.zeros_like(x)
                for e in idx.unique().tolist():
                    rows, ks = (idx == e).nonzero(as_tuple=True)
                    pe = f + f"experts.{e}."
                    y.index_add_(0, rows, swiglu(x[rows], self._expert(pe, "w1"), self._expert(pe, "w3"),
                                                 self._expert(pe, "w2"), cfg.swiglu_limit) * wts[rows, ks, None])
                if cfg.num_shared_experts:
                    y = y + swiglu(x, self._w(f + "shared_experts.w1.weight"), self._w(f + "shared_experts.w3.weight"),
                                   self._w(f + "shared_experts.w2.weight"))
            h = h + y
        return rms_norm(h, self._w("norm.weight"), cfg.rms_norm_eps) @ self._w("head.weight").t()

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new_tokens: int):
        ids = prompt.clone()
        toks, rows = [], []
        for _ in range(max_new_tokens):
            logits = self.forward(ids)[-1]
            rows.append(logits)
            toks.append(int(logits.argmax()))
            ids = torch.cat([ids, torch.tensor([toks[-1]], dtype=ids.dtype)])
        return toks, torch.stack(rows)
