"""fp32 oracle for the Qwen-style hybrid model: plain PyTorch, whole-sequence forward, no caches.

Math follows the reference's engine (cpp_engine/engine/qwen_engine.cpp:2297-3313) with the
chunk-free token recurrence for Gated DeltaNet (cpp_engine/backends/cuda/kernels/qwen_half_ops.cu:2282-2347).
Intermediate activations are rounded to bf16 where the GPU runtime stores them in bf16, so the
comparison isolates kernel error from storage rounding.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ...formats import fp8 as fp8fmt
from ...ops.attention import attention_ref, rope_ref
from ...ops.basic import conv_silu_ref, gated_rmsnorm_ref, gdn_gates_ref, rmsnorm_ref
from ...ops.gdn import recurrent_ref


def _r(x):  # storage rounding
    return x.to(torch.bfloat16).float()


class QwenHybridRef:
    def __init__(self, cfg, state):
        self.cfg = cfg
        self.capture_layers: tuple[int, ...] = ()          # layers whose output hidden state ``forward`` keeps (drafter taps)
        raw = dict(state)
        self.p = {}
        for k, v in raw.items():
            if k.endswith((".weight_scale_inv", ".weight_scale", ".weight_global_scale", ".input_global_scale")):
                continue
            if k.endswith(".weight_packed"):                       # NVFP4 (formats/nvfp4.py)
                from ...formats import nvfp4
                base = k[:-len(".weight_packed")]
                self.p[base + ".weight"] = nvfp4.dequantize(v.cpu(), raw[base + ".weight_scale"].cpu(),
                                                            raw[base + ".weight_global_scale"].cpu())
            elif v.dtype == torch.float8_e4m3fn:
                self.p[k] = fp8fmt.dequantize_block128(v, raw[k + "_scale_inv"])
            else:
                self.p[k] = v.float()

    def lin(self, x, name):
        return x @ self.p[name + ".weight"].t()

    @torch.no_grad()
    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [T] -> logits [T, vocab] fp32 (single sequence from position 0)."""
        cfg, p = self.cfg, self.p
        t = ids.numel()
        eps = cfg.rms_norm_eps
        h = p["model.language_model.embed_tokens.weight"][ids.long()]
        pos = torch.arange(t, device=ids.device)
        inv = (1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.rotary_dim, 2, dtype=torch.float64) / cfg.rotary_dim))).float().to(ids.device)
        taps = {}
        for i, lt in enumerate(cfg.layer_types):
            pre = f"model.language_model.layers.{i}."
            x = _r(rmsnorm_ref(h, p[pre + "input_layernorm.weight"], eps, True))
            if lt == "linear_attention":
                a = pre + "linear_attn."
                hk, hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
                qkv = _r(self.lin(x, a + "in_proj_qkv"))
                z = _r(self.lin(x, a + "in_proj_z"))
                av, bv = _r(self.lin(x, a + "in_proj_a")), _r(self.lin(x, a + "in_proj_b"))
                conv_w = p[a + "conv1d.weight"].reshape(qkv.shape[1], -1)
                mixed, _ = conv_silu_ref(qkv, conv_w, torch.zeros(conv_w.shape[1] - 1, qkv.shape[1], device=ids.device))
                mixed = _r(mixed)
                g, beta = gdn_gates_ref(av, bv, p[a + "A_log"], p[a + "dt_bias"])
                q = mixed[:, :hk * 128].view(t, hk, 128)
                k = mixed[:, hk * 128:2 * hk * 128].view(t, hk, 128)
                v = mixed[:, 2 * hk * 128:].view(t, hv, 128)
                core, _ = recurrent_ref(q, k, v, g, beta, torch.zeros(hv, 128, 128, device=ids.device))
                y = _r(gated_rmsnorm_ref(_r(core), z.view(t, hv, 128), p[a + "norm.weight"], eps))
                d = _r(self.lin(y.reshape(t, -1), a + "out_proj"))
            else:
                a = pre + "self_attn."
                hq, hkv = cfg.num_attention_heads, cfg.num_key_value_heads
                qg = _r(self.lin(x, a + "q_proj")).view(t, hq, -1)
                q, gate = (qg[..., :128], qg[..., 128:]) if cfg.attn_output_gate else (qg, None)
                k = _r(self.lin(x, a + "k_proj")).view(t, hkv, 128)
                v = _r(self.lin(x, a + "v_proj")).view(t, hkv, 128)
                q = _r(rope_ref(rmsnorm_ref(q, p[a + "q_norm.weight"], eps, True), pos, inv, cfg.rotary_dim))
                k = _r(rope_ref(rmsnorm_ref(k, p[a + "k_norm.weight"], eps, True), pos, inv, cfg.rotary_dim))
                o = _r(attention_ref(q, k, v, 0, gate))
                d = _r(self.lin(o.reshape(t, -1), a + "o_proj"))
            h = _r(h + d)
            x = _r(rmsnorm_ref(h, p[pre + "post_attention_layernorm.weight"], eps, True))
            gu = torch.cat([_r(self.lin(x, pre + "mlp.gate_proj")), _r(self.lin(x, pre + "mlp.up_proj"))], -1)
            g_, u_ = gu.chunk(2, -1)
            act = _r(F.silu(g_) * u_)
            h = _r(h + _r(self.lin(act, pre + "mlp.down_proj")))
            if i in self.capture_layers:
                taps[i] = h
        if self.capture_layers:                                # [T, len(capture_layers) * H], in the order asked for
            self.last_taps = torch.cat([taps[i] for i in self.capture_layers], -1)
        x = _r(rmsnorm_ref(h, p["model.language_model.norm.weight"], eps, True))
        self.last_hidden = x                                   # final-normed trunk output [T, H]: what the MTP head consumes
        return x @ p["lm_head.weight"].t()

    @torch.no_grad()
    def mtp_forward(self, next_ids: torch.Tensor, hidden: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """Multi-token-prediction head over a whole sequence: row i fuses the embedding of ``next_ids[i]`` (the token
        after position i) with ``hidden[i]`` and predicts the token after that.  Returns (logits [T, vocab], the head's
        normalised hidden [T, H], which a second recursive step would consume in place of ``hidden``).
        Reference behaviour: cpp_engine/engine/qwen_engine.cpp:3680-3730 (embedding and hidden normalised separately,
        concatenated, ``mtp.fc``, one full-attention decoder layer, ``mtp.norm``, shared lm_head)."""
        cfg, p = self.cfg, self.p
        t, eps = next_ids.numel(), cfg.rms_norm_eps
        e = _r(rmsnorm_ref(p["model.language_model.embed_tokens.weight"][next_ids.long()], p["mtp.pre_fc_norm_embedding.weight"], eps, True))
        hn = _r(rmsnorm_ref(hidden.float(), p["mtp.pre_fc_norm_hidden.weight"], eps, True))
        h = _r(self.lin(torch.cat([e, hn], -1), "mtp.fc"))
        pos = torch.arange(t, device=next_ids.device)
        inv = (1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.rotary_dim, 2, dtype=torch.float64) / cfg.rotary_dim))).float().to(next_ids.device)
        pre, a = "mtp.layers.0.", "mtp.layers.0.self_attn."
        hq, hkv = cfg.num_attention_heads, cfg.num_key_value_heads
        x = _r(rmsnorm_ref(h, p[pre + "input_layernorm.weight"], eps, True))
        qg = _r(self.lin(x, a + "q_proj")).view(t, hq, -1)
        q, gate = (qg[..., :128], qg[..., 128:]) if cfg.attn_output_gate else (qg, None)
        k = _r(self.lin(x, a + "k_proj")).view(t, hkv, 128)
        v = _r(self.lin(x, a + "v_proj")).view(t, hkv, 128)
        q = _r(rope_ref(rmsnorm_ref(q, p[a + "q_norm.weight"], eps, True), pos, inv, cfg.rotary_dim))
        k = _r(rope_ref(rmsnorm_ref(k, p[a + "k_norm.weight"], eps, True), pos, inv, cfg.rotary_dim))
        h = _r(h + _r(self.lin(_r(attention_ref(q, k, v, 0, gate)).reshape(t, -1), a + "o_proj")))
        x = _r(rmsnorm_ref(h, p[pre + "post_attention_layernorm.weight"], eps, True))
        act = _r(F.silu(_r(self.lin(x, pre + "mlp.gate_proj"))) * _r(self.lin(x, pre + "mlp.up_proj")))
        h = _r(h + _r(self.lin(act, pre + "mlp.down_proj")))
        out = _r(rmsnorm_ref(h, p["mtp.norm.weight"], eps, True))
        return out @ p["lm_head.weight"].t(), out


def synth_mtp_state(cfg, seed: int = 0, std: float = 0.05, fp8_linears: bool = False):
    """(name, tensor) pairs of a random MTP head for ``cfg``: bf16 vectors, matrices bf16 or FP8 block-128."""
    g = torch.Generator().manual_seed(seed + 4242)
    h, inter, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    qd, kvd = cfg.num_attention_heads * d, cfg.num_key_value_heads * d
    out = []
    vec = lambda n, k: out.append((n, (1.0 + 0.05 * torch.randn(k, generator=g)).to(torch.bfloat16)))

    def lin(base, n, k):
        w = torch.randn(n, k, generator=g) * std
        if fp8_linears:
            q, s = fp8fmt.quantize_block128(w)
            out.extend([(base + ".weight", q), (base + ".weight_scale_inv", s)])
        else:
            out.append((base + ".weight", w.to(torch.bfloat16)))

    vec("mtp.pre_fc_norm_embedding.weight", h); vec("mtp.pre_fc_norm_hidden.weight", h); vec("mtp.norm.weight", h)
    lin("mtp.fc", h, 2 * h)
    p = "mtp.layers.0."
    vec(p + "input_layernorm.weight", h); vec(p + "post_attention_layernorm.weight", h)
    lin(p + "self_attn.q_proj", qd * (2 if cfg.attn_output_gate else 1), h)
    lin(p + "self_attn.k_proj", kvd, h); lin(p + "self_attn.v_proj", kvd, h); lin(p + "self_attn.o_proj", h, qd)
    vec(p + "self_attn.q_norm.weight", d); vec(p + "self_attn.k_norm.weight", d)
    lin(p + "mlp.gate_proj", inter, h); lin(p + "mlp.up_proj", inter, h); lin(p + "mlp.down_proj", h, inter)
    return out
