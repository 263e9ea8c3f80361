"""DeepSeek / GLM-style decoder family: Multi-head Latent Attention (+ optional sparse top-k indexer)
with routed-expert MoE layers (+ shared expert, + leading dense layers).

One config-driven runtime covers
* the tiny CPU model used for parity checks (fp32 activations, FP4 E2M1 experts executed by the
  host kernels in ``csrc/cpu/cpu_moe_fp4.cpp`` straight from the packed bytes),
* DeepSeek-V4-Flash-shaped and GLM-5.2-shaped models (MLA with a latent KV cache, lightning
  indexer selecting the top-k keys per query, routed experts with sigmoid / softmax /
  sqrt-softplus scoring and selection bias).

Attention runs in the *absorbed* form: the cache stores, per token, the normalised latent
``c_kv`` (kv_lora_rank) and the shared rotary key (qk_rope_dim); queries are projected into latent
space (``q_nope W_uk``), scores are taken against the latent cache, and the value up-projection is
applied after the softmax-weighted sum.  The fp32 oracle in ``reference_cpu/mla_moe_ref.py``
uses the expanded per-head K/V form instead, so agreement between the two checks the algebra.

Reference behaviour covered: MLA of the GLM runtime (src/models/glm_dsa/architecture.py:263-406),
indexer scoring of the DeepSeek-V4 runtime (src/models/deepseek_v4/runtime.py:1112-1288, restated
for MLA keys), gate / expert / shared-expert semantics (src/models/deepseek_v4/runtime.py:1662-1760,
3664-4274), expert-range sharding over ranks (:2693-2694).
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Iterator

import torch
import torch.nn.functional as F

from ..formats import fp4 as fp4fmt


# ------------------------------------------------------------------ config
@dataclass
class MlaMoeConfig:
    vocab_size: int = 129280
    hidden_size: int = 4096
    num_layers: int = 43
    first_dense_layers: int = 3
    dense_intermediate: int = 12288
    # MLA
    q_lora_rank: int = 1024            # 0 = direct q projection
    kv_lora_rank: int = 512
    num_heads: int = 64
    qk_nope_dim: int = 128
    qk_rope_dim: int = 64
    v_head_dim: int = 128
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    # sparse indexer (0 heads = dense attention over the whole cache)
    index_heads: int = 64
    index_dim: int = 128
    index_topk: int = 2048
    # MoE
    num_experts: int = 256
    experts_per_token: int = 6
    num_shared_experts: int = 1
    expert_intermediate: int = 2048
    score_func: str = "sqrtsoftplus"   # softmax | sigmoid | sqrtsoftplus
    route_scale: float = 1.5
    norm_topk: bool = True
    swiglu_limit: float = 0.0
    expert_format: str = "fp4"         # fp4 | bf16
    mtp_layers: int = 0

    @property
    def qk_head_dim(self) -> int:
        return self.qk_nope_dim + self.qk_rope_dim

    # config.json in the spelling of the DeepSeek inference configs (configs/config.json of the reference:
    # dim, n_layers, n_dense_layers, n_heads, inter_dim, moe_inter_dim, n_routed_experts, n_shared_experts,
    # n_activated_experts, route_scale, q_lora_rank, kv_lora_rank, qk_nope_head_dim, qk_rope_head_dim, v_head_dim,
    # index_n_heads, index_head_dim, index_topk, score_func, expert_dtype, n_mtp_layers)
    _JSON = {"vocab_size": "vocab_size", "hidden_size": "dim", "num_layers": "n_layers", "first_dense_layers": "n_dense_layers",
             "dense_intermediate": "inter_dim", "q_lora_rank": "q_lora_rank", "kv_lora_rank": "kv_lora_rank",
             "num_heads": "n_heads", "qk_nope_dim": "qk_nope_head_dim", "qk_rope_dim": "qk_rope_head_dim",
             "v_head_dim": "v_head_dim", "rope_theta": "rope_theta", "rms_norm_eps": "rms_norm_eps",
             "index_heads": "index_n_heads", "index_dim": "index_head_dim", "index_topk": "index_topk",
             "num_experts": "n_routed_experts", "experts_per_token": "n_activated_experts",
             "num_shared_experts": "n_shared_experts", "expert_intermediate": "moe_inter_dim", "score_func": "score_func",
             "route_scale": "route_scale", "norm_topk": "norm_topk_prob", "swiglu_limit": "swiglu_limit",
             "expert_format": "expert_dtype", "mtp_layers": "n_mtp_layers"}

    def to_json(self) -> dict:
        d = {j: getattr(self, f) for f, j in self._JSON.items()}
        d["model_type"] = "deepseek_mla_moe"
        return d

    @staticmethod
    def is_mla_moe_json(d: dict) -> bool:
        """Does a config.json describe this family (DeepSeek inference spelling)?"""
        return isinstance(d, dict) and "n_routed_experts" in d and "kv_lora_rank" in d and "dim" in d

    @staticmethod
    def from_json(d: dict) -> "MlaMoeConfig":
        kw = {}
        base = MlaMoeConfig()
        for f, j in MlaMoeConfig._JSON.items():
            if j in d and d[j] is not None:
                kw[f] = type(getattr(base, f))(d[j])
        if "index_n_heads" not in d:              # a checkpoint without the sparse indexer
            kw.update(index_heads=0, index_dim=0, index_topk=0)
        return MlaMoeConfig(**kw)

    @staticmethod
    def tiny_cpu() -> "MlaMoeConfig":
        """2 layers, hidden 256, vocab 1024, MLA (q_lora 128, kv_lora 64, 4 heads, 32 + 16, v 32), 8 routed
        experts top-2 + 1 shared (intermediate 128), no indexer, no dense layers."""
        return MlaMoeConfig(vocab_size=1024, hidden_size=256, num_layers=2, first_dense_layers=0, dense_intermediate=512,
                            q_lora_rank=128, kv_lora_rank=64, num_heads=4, qk_nope_dim=32, qk_rope_dim=16, v_head_dim=32,
                            index_heads=0, index_dim=0, index_topk=0, num_experts=8, experts_per_token=2,
                            num_shared_experts=1, expert_intermediate=128)

    @staticmethod
    def deepseek_v4_flash_shaped() -> "MlaMoeConfig":
        return MlaMoeConfig()

    @staticmethod
    def glm_5_2_shaped() -> "MlaMoeConfig":
        return MlaMoeConfig(vocab_size=154880, hidden_size=6144, num_layers=78, first_dense_layers=3,
                            dense_intermediate=12288, q_lora_rank=2048, kv_lora_rank=512, num_heads=64,
                            qk_nope_dim=192, qk_rope_dim=64, v_head_dim=256, index_heads=32, index_dim=128,
                            index_topk=2048, num_experts=256, experts_per_token=8, expert_intermediate=2048,
                            score_func="sigmoid", route_scale=2.5, expert_format="bf16")


# ------------------------------------------------------- synthetic checkpoints
def tensor_specs(cfg: MlaMoeConfig) -> list[tuple[str, tuple[int, ...], str]]:
    """(name, shape, kind); kind: w (N(0, .02) bf16) | norm (ones-ish bf16) | bias (fp32) | expert (FP4 or bf16)."""
    h = cfg.hidden_size
    out: list[tuple[str, tuple[int, ...], str]] = [("embed.weight", (cfg.vocab_size, h), "w"), ("norm.weight", (h,), "norm"),
                                                   ("head.weight", (cfg.vocab_size, h), "w")]
    qd = cfg.num_heads * cfg.qk_head_dim
    for i in range(cfg.num_layers + cfg.mtp_layers):
        p = f"layers.{i}." if i < cfg.num_layers else f"mtp.{i - cfg.num_layers}."
        if i >= cfg.num_layers:
            out += [(p + "e_proj.weight", (h, h), "w"), (p + "h_proj.weight", (h, h), "w"),
                    (p + "enorm.weight", (h,), "norm"), (p + "hnorm.weight", (h,), "norm")]
        out += [(p + "attn_norm.weight", (h,), "norm"), (p + "ffn_norm.weight", (h,), "norm")]
        a = p + "attn."
        if cfg.q_lora_rank > 0:
            out += [(a + "wq_a.weight", (cfg.q_lora_rank, h), "w"), (a + "q_norm.weight", (cfg.q_lora_rank,), "norm"),
                    (a + "wq_b.weight", (qd, cfg.q_lora_rank), "w")]
        else:
            out += [(a + "wq.weight", (qd, h), "w")]
        out += [(a + "wkv_a.weight", (cfg.kv_lora_rank + cfg.qk_rope_dim, h), "w"),
                (a + "kv_norm.weight", (cfg.kv_lora_rank,), "norm"),
                (a + "wkv_b.weight", (cfg.num_heads * (cfg.qk_nope_dim + cfg.v_head_dim), cfg.kv_lora_rank), "w"),
                (a + "wo.weight", (h, cfg.num_heads * cfg.v_head_dim), "w")]
        if cfg.index_heads > 0:
            qin = cfg.q_lora_rank if cfg.q_lora_rank > 0 else h
            out += [(a + "indexer.wq_b.weight", (cfg.index_heads * cfg.index_dim, qin), "w"),
                    (a + "indexer.wk.weight", (cfg.index_dim, h), "w"),
                    (a + "indexer.k_norm.weight", (cfg.index_dim,), "norm"),
                    (a + "indexer.weights_proj.weight", (cfg.index_heads, h), "w")]
        f = p + "ffn."
        if i < cfg.first_dense_layers:
            d = cfg.dense_intermediate
            out += [(f + "w1.weight", (d, h), "w"), (f + "w3.weight", (d, h), "w"), (f + "w2.weight", (h, d), "w")]
        else:
            e_i = cfg.expert_intermediate
            out += [(f + "gate.weight", (cfg.num_experts, h), "w"), (f + "gate.bias", (cfg.num_experts,), "bias")]
            for e in range(cfg.num_experts):
                out += [(f + f"experts.{e}.w1.weight", (e_i, h), "expert"), (f + f"experts.{e}.w3.weight", (e_i, h), "expert"),
                        (f + f"experts.{e}.w2.weight", (h, e_i), "expert")]
            if cfg.num_shared_experts:
                s_i = e_i * cfg.num_shared_experts
                out += [(f + "shared_experts.w1.weight", (s_i, h), "w"), (f + "shared_experts.w3.weight", (s_i, h), "w"),
                        (f + "shared_experts.w2.weight", (h, s_i), "w")]
    return out


def synth_state(cfg: MlaMoeConfig, seed: int = 0, device="cpu", std: float = 0.02,
                expert_range: tuple[int, int] | None = None, expert_pool: int | None = None,
                layer_range: tuple[int, int] | None = None) -> Iterator[tuple[str, torch.Tensor]]:
    """Seeded random-init checkpoint tensors in checkpoint dtypes (FP4 experts come as ``.weight`` packed uint8
    plus ``.scale`` E8M0 uint8).  For full-size benchmarks a rank can restrict generation to the experts and layers
    it holds, and draw only ``expert_pool`` distinct experts per layer (expert e re-uses the tensors of e % pool)."""
    gen = torch.Generator(device=device)
    pool_cache: dict[str, list] = {}
    for idx, (name, shape, kind) in enumerate(tensor_specs(cfg)):
        if layer_range is not None and name.startswith("layers."):
            li = int(name.split(".")[1])
            if not (layer_range[0] <= li < layer_range[1]):
                continue
        if kind == "expert" and ".experts." in name:
            head, rest = name.split(".experts.")
            e = int(rest.split(".")[0])
            if expert_range is not None and not (expert_range[0] <= e < expert_range[1]):
                continue
            if expert_pool:
                import zlib
                key = head + ".experts." + str(e % expert_pool) + "." + rest.split(".", 1)[1]
                if key not in pool_cache:
                    gen.manual_seed(seed * 1_000_003 + zlib.crc32(key.encode()))
                    w = torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std
                    if cfg.expert_format == "fp4":
                        q_, s_ = fp4fmt.quantize(w)
                        pool_cache[key] = [("weight", q_), ("scale", s_)]
                    else:
                        pool_cache[key] = [("weight", w.bfloat16())]
                for suffix, t in pool_cache[key]:
                    yield name[:-len("weight")] + suffix, t
                continue
        gen.manual_seed(seed * 1_000_003 + idx)
        if kind == "w":
            yield name, (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std).bfloat16()
        elif kind == "norm":
            yield name, (1.0 + torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * 0.05).bfloat16()
        elif kind == "bias":
            yield name, torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * 0.01
        elif kind == "expert":
            w = torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std
            if cfg.expert_format == "fp4":
                q, s = fp4fmt.quantize(w)
                out = [("weight", q), ("scale", s)]
            else:
                out = [("weight", w.bfloat16())]
            for suffix, t in out:
                yield name[:-len("weight")] + suffix, t
        else:
            raise ValueError(kind)


# ------------------------------------------------------------------ host kernels
_cpu_lib = None


def cpu_lib() -> ctypes.CDLL:
    global _cpu_lib
    if _cpu_lib is None:
        path = Path(__file__).resolve().parent.parent / "lib" / "libb200_cpu.so"
        if not path.exists():
            from .. import build as _build

            _build.build_cpu()
        _cpu_lib = ctypes.CDLL(str(path))
    return _cpu_lib


def cpu_moe_fp4(x: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, w13, s13, w2, s2, inter: int,
                swiglu_limit: float = 0.0, threads: int = 0) -> torch.Tensor:
    """Routed FP4 experts on the host. x [T, H] fp32; idx [T, K] int32; wts [T, K] fp32; returns [T, H] fp32."""
    t, h = x.shape
    out = torch.zeros(t, h, dtype=torch.float32)
    x = x.contiguous().float()
    idx = idx.contiguous().to(torch.int32)
    wts = wts.contiguous().float()
    p = lambda a: ctypes.c_void_p(a.data_ptr())
    rc = cpu_lib().b200_cpu_moe_fp4_forward(p(x), t, h, p(idx), p(wts), idx.shape[1], p(w13), p(s13), p(w2), p(s2),
                                            w13.shape[0], inter, ctypes.c_float(swiglu_limit), p(out), threads)
    if rc != 0:
        raise RuntimeError("cpu_moe_fp4_forward rejected its arguments")
    return out


_iq2xxs_sent = False


def cpu_gguf_linear(x: torch.Tensor, raw: torch.Tensor, ggml_type: int, threads: int = 0) -> torch.Tensor:
    """y [T, N] = x [T, K] @ W^T on the host with W as raw GGUF blocks uint8 [N, row_bytes] (Q8_0 = 8, Q2_K = 10, IQ2_XXS = 16)."""
    x = x.contiguous().float()
    raw = raw.contiguous()
    t, k = x.shape
    n = raw.shape[0]
    y = torch.empty(t, n, dtype=torch.float32)
    p = lambda a: ctypes.c_void_p(a.data_ptr())
    global _iq2xxs_sent
    if int(ggml_type) == 16 and not _iq2xxs_sent:                 # hand the codebook to the library once
        from ..formats.gguf import quant as _q
        tb = _q.tables("cpu")
        grid, ks = tb["iq2xxs"].contiguous().float(), tb["ksigns"].contiguous()
        cpu_lib().b200_cpu_gguf_set_iq2xxs_tables(p(grid), p(ks))
        _iq2xxs_sent = True
    rc = cpu_lib().b200_cpu_gguf_linear(int(ggml_type), p(x), t, k, p(raw), n, p(y), threads)
    if rc != 0:
        raise RuntimeError("cpu_gguf_linear: unsupported type" if rc == -2 else "cpu_gguf_linear rejected its arguments")
    return y


def cpu_moe_gguf(x: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, gate_raw: torch.Tensor, up_raw: torch.Tensor,
                 down_raw: torch.Tensor, gate_type: int, down_type: int, swiglu_limit: float = 0.0, threads: int = 0) -> torch.Tensor:
    """Routed experts on the host straight from stacked raw GGUF tensors: gate_raw / up_raw uint8 [E, I, row_bytes(H)],
    down_raw [E, H, row_bytes(I)].  Tokens are grouped by expert, so each active expert's blocks are walked once.
    x [T, H] fp32, idx [T, K] (negative = unused), wts [T, K]; returns [T, H] fp32."""
    x = x.contiguous().float()
    out = torch.zeros_like(x)
    idx = idx.long()
    for e in idx[idx >= 0].unique().tolist():
        rows, slot = (idx == e).nonzero(as_tuple=True)
        xe = x[rows]
        g = cpu_gguf_linear(xe, gate_raw[e], gate_type, threads)
        u = cpu_gguf_linear(xe, up_raw[e], gate_type, threads)
        if swiglu_limit > 0:
            g, u = g.clamp(max=swiglu_limit), u.clamp(-swiglu_limit, swiglu_limit)
        h = torch.nn.functional.silu(g) * u * wts[rows, slot].float()[:, None]
        out.index_add_(0, rows, cpu_gguf_linear(h, down_raw[e], down_type, threads))
    return out


def quantize_rows_int8(w: torch.Tensor, threads: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-row symmetric INT8: w [..., N, K] fp32 -> (int8 [..., N, K], fp32 scale [..., N]), scale = max|row| / 127."""
    w = w.contiguous().float()
    n, k = int(w.numel() // w.shape[-1]), w.shape[-1]
    q = torch.empty(w.shape, dtype=torch.int8)
    s = torch.empty(w.shape[:-1], dtype=torch.float32)
    p = lambda a: ctypes.c_void_p(a.data_ptr())
    if cpu_lib().b200_cpu_quantize_rows_int8(p(w), n, k, p(q), p(s), threads) != 0:
        raise RuntimeError("cpu_quantize_rows_int8 rejected its arguments")
    return q, s


def cpu_moe_int8(x: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, w13: torch.Tensor, s13: torch.Tensor, w2: torch.Tensor,
                 s2: torch.Tensor, swiglu_limit: float = 0.0, threads: int = 0) -> torch.Tensor:
    """Routed INT8 (W8A8) experts on the host.  x [T, H] fp32; idx [T, K] int32; wts [T, K] fp32; w13 int8 [E, 2I, H] with
    s13 [E, 2I]; w2 int8 [E, H, I] with s2 [E, H]; returns [T, H] fp32."""
    t, h = x.shape
    e, two_i, _ = w13.shape
    assert w13.dtype == torch.int8 and w2.dtype == torch.int8 and w2.shape == (e, h, two_i // 2)
    out = torch.zeros(t, h, dtype=torch.float32)
    x, idx, wts = x.contiguous().float(), idx.contiguous().to(torch.int32), wts.contiguous().float()
    w13, w2, s13, s2 = w13.contiguous(), w2.contiguous(), s13.contiguous().float(), s2.contiguous().float()
    p = lambda a: ctypes.c_void_p(a.data_ptr())
    rc = cpu_lib().b200_cpu_moe_int8_forward(p(x), t, h, p(idx), p(wts), idx.shape[1], p(w13), p(s13), p(w2), p(s2), e,
                                             two_i // 2, ctypes.c_float(swiglu_limit), p(out), threads)
    if rc != 0:
        raise RuntimeError("cpu_moe_int8_forward rejected its arguments")
    return out


# ------------------------------------------------------------------ shared math
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()


def rope_interleaved(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate adjacent pairs (x[2i], x[2i+1]) of the last dim. x [T, ..., D]; positions [T]."""
    d = x.shape[-1]
    inv = theta ** (-torch.arange(0, d, 2, dtype=torch.float32, device=x.device) / d)
    ang = positions.float()[:, None] * inv[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [d // 2]
    cos, sin = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    x1, x2 = x[..., 0::2].float(), x[..., 1::2].float()
    return torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), -1).flatten(-2)


def route(cfg: MlaMoeConfig, x: torch.Tensor, gate_w: torch.Tensor, gate_b: torch.Tensor | None):
    """Scores, top-k selection with bias, weights from the unbiased scores (normalised, scaled)."""
    s = x.float() @ gate_w.float().t()
    if cfg.score_func == "softmax":
        s = s.softmax(-1)
    elif cfg.score_func == "sigmoid":
        s = s.sigmoid()
    else:
        s = F.softplus(s).sqrt()
    sel = s + gate_b.float() if gate_b is not None else s
    idx = sel.topk(cfg.experts_per_token, -1).indices
    w = s.gather(1, idx)
    if cfg.score_func != "softmax" and cfg.norm_topk:
        w = w / w.sum(-1, keepdim=True)
    return w * cfg.route_scale, idx


def swiglu(x, w1, w3, w2, limit: float = 0.0):
    g, u = x @ w1.t(), x @ w3.t()
    if limit > 0:
        u = u.clamp(-limit, limit)
        g = g.clamp(max=limit)
    return (F.silu(g) * u) @ w2.t()


# ------------------------------------------------------------------ weights
@dataclass
class MlaLayer:
    attn_norm: torch.Tensor
    ffn_norm: torch.Tensor
    wq_a: torch.Tensor | None
    q_norm: torch.Tensor | None
    wq_b: torch.Tensor
    wkv_a: torch.Tensor
    kv_norm: torch.Tensor
    w_uk: torch.Tensor            # [heads, nope, kv_lora]
    w_uv: torch.Tensor            # [heads, v, kv_lora]
    wo: torch.Tensor
    idx_wq: torch.Tensor | None = None
    idx_wk: torch.Tensor | None = None
    idx_knorm: torch.Tensor | None = None
    idx_wproj: torch.Tensor | None = None
    dense: tuple | None = None    # (w1, w3, w2)
    gate_w: torch.Tensor | None = None
    gate_b: torch.Tensor | None = None
    shared: tuple | None = None
    # routed experts of this rank: FP4 -> (w13 [E, 2I, H/2], s13, w2 [E, H, I/2], s2); bf16 -> (w1, w3, w2) stacks
    experts: tuple | None = None


class MlaMoeWeights:
    """Weights on ``device`` with routed experts [expert_lo, expert_hi) of this rank stacked per layer."""

    def __init__(self, cfg: MlaMoeConfig, state: Iterator[tuple[str, torch.Tensor]], device="cpu", ep_rank: int = 0,
                 ep_world: int = 1, dtype=torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        per = cfg.num_experts // ep_world
        assert per * ep_world == cfg.num_experts
        self.expert_lo, self.expert_hi = ep_rank * per, (ep_rank + 1) * per
        sd: dict[str, torch.Tensor] = {}
        for k, v in state:
            if ".experts." in k:
                e = int(k.split(".experts.")[1].split(".")[0])
                if not (self.expert_lo <= e < self.expert_hi):
                    continue
            sd[k] = v
        d = lambda t: t.to(self.device, dtype)
        self.embed = d(sd["embed.weight"])
        self.norm = d(sd["norm.weight"])
        self.head = d(sd["head.weight"])
        self.layers: list[MlaLayer] = []
        for i in range(cfg.num_layers):
            self.layers.append(self._layer(sd, f"layers.{i}.", i < cfg.first_dense_layers))

    def _layer(self, sd, p: str, dense: bool) -> MlaLayer:
        cfg = self.cfg
        d = lambda t: t.to(self.device, self.dtype)
        a = p + "attn."
        wkv_b = d(sd[a + "wkv_b.weight"]).view(cfg.num_heads, cfg.qk_nope_dim + cfg.v_head_dim, cfg.kv_lora_rank)
        lw = MlaLayer(
            attn_norm=d(sd[p + "attn_norm.weight"]), ffn_norm=d(sd[p + "ffn_norm.weight"]),
            wq_a=d(sd[a + "wq_a.weight"]) if cfg.q_lora_rank > 0 else None,
            q_norm=d(sd[a + "q_norm.weight"]) if cfg.q_lora_rank > 0 else None,
            wq_b=d(sd[a + ("wq_b.weight" if cfg.q_lora_rank > 0 else "wq.weight")]),
            wkv_a=d(sd[a + "wkv_a.weight"]), kv_norm=d(sd[a + "kv_norm.weight"]),
            w_uk=wkv_b[:, :cfg.qk_nope_dim].contiguous(), w_uv=wkv_b[:, cfg.qk_nope_dim:].contiguous(),
            wo=d(sd[a + "wo.weight"]))
        if cfg.index_heads > 0:
            lw.idx_wq, lw.idx_wk = d(sd[a + "indexer.wq_b.weight"]), d(sd[a + "indexer.wk.weight"])
            lw.idx_knorm, lw.idx_wproj = d(sd[a + "indexer.k_norm.weight"]), d(sd[a + "indexer.weights_proj.weight"])
        f = p + "ffn."
        if dense:
            lw.dense = (d(sd[f + "w1.weight"]), d(sd[f + "w3.weight"]), d(sd[f + "w2.weight"]))
            return lw
        lw.gate_w, lw.gate_b = d(sd[f + "gate.weight"]), sd[f + "gate.bias"].to(self.device, torch.float32)
        if cfg.num_shared_experts:
            lw.shared = tuple(d(sd[f + f"shared_experts.{n}.weight"]) for n in ("w1", "w3", "w2"))
        es = range(self.expert_lo, self.expert_hi)
        if cfg.expert_format == "fp4":
            cat = lambda n, suf: torch.stack([sd[f + f"experts.{e}.{n}.{suf}"] for e in es]).to(self.device)
            w13 = torch.cat([cat("w1", "weight"), cat("w3", "weight")], 1).contiguous()
            s13 = torch.cat([cat("w1", "scale"), cat("w3", "scale")], 1).contiguous()
            lw.experts = (w13, s13, cat("w2", "weight").contiguous(), cat("w2", "scale").contiguous())
        else:
            lw.experts = tuple(torch.stack([d(sd[f + f"experts.{e}.{n}.weight"]) for e in es]) for n in ("w1", "w3", "w2"))
        return lw


# ------------------------------------------------------------------ runtime
@dataclass
class MlaSeq:
    length: int = 0


class MlaMoeRuntime:
    """Incremental (prefill + decode) forward with a latent KV cache per layer.

    This class is the host execution path: dense algebra through PyTorch on ``weights.device``, FP4 routed
    experts through the packed-byte host kernels.  ``comm`` (optional) sums the routed-expert output over
    expert-parallel ranks."""

    def __init__(self, cfg: MlaMoeConfig, weights: MlaMoeWeights, max_context: int = 4096, comm=None):
        self.cfg, self.w, self.device = cfg, weights, weights.device
        self.comm = comm
        self.max_context = max_context
        n = cfg.num_layers
        self.ckv = torch.zeros(n, max_context, cfg.kv_lora_rank, dtype=torch.float32, device=self.device)
        self.kpe = torch.zeros(n, max_context, cfg.qk_rope_dim, dtype=torch.float32, device=self.device)
        self.kidx = torch.zeros(n, max_context, max(1, cfg.index_dim), dtype=torch.float32, device=self.device)
        self.length = 0

    def reset(self) -> None:
        self.length = 0

    # ---- attention
    def _indexer_select(self, lw: MlaLayer, i: int, x: torch.Tensor, qin: torch.Tensor, pos: torch.Tensor, end: int):
        """Top-k key positions per query row (None = attend to everything). score[t, s] = sum_h relu(q_h . k_s) w_h."""
        cfg = self.cfg
        if cfg.index_heads <= 0 or end <= cfg.index_topk:
            # the key is still written so later steps can select
            if cfg.index_heads > 0:
                k = rms_norm(x @ lw.idx_wk.t(), lw.idx_knorm, cfg.rms_norm_eps)
                self.kidx[i, pos] = k
            return None
        t = x.shape[0]
        k = rms_norm(x @ lw.idx_wk.t(), lw.idx_knorm, cfg.rms_norm_eps)
        self.kidx[i, pos] = k
        q = (qin @ lw.idx_wq.t()).view(t, cfg.index_heads, cfg.index_dim)
        hw = (x @ lw.idx_wproj.t()) * cfg.index_heads ** -0.5
        sc = torch.einsum("thd,sd->ths", q, self.kidx[i, :end]).relu()
        sc = (sc * hw[:, :, None]).sum(1) * cfg.index_dim ** -0.5
        causal = torch.arange(end, device=x.device)[None, :] <= pos[:, None]
        sc = sc.masked_fill(~causal, float("-inf"))
        return sc.topk(cfg.index_topk, -1).indices          # [T, topk]; -inf entries are masked again below

    def _attention(self, lw: MlaLayer, i: int, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        t = x.shape[0]
        start, end = int(pos[0]), int(pos[-1]) + 1
        if cfg.q_lora_rank > 0:
            qin = rms_norm(x @ lw.wq_a.t(), lw.q_norm, cfg.rms_norm_eps)
        else:
            qin = x
        q = (qin @ lw.wq_b.t()).view(t, cfg.num_heads, cfg.qk_head_dim)
        q_nope, q_pe = q[..., :cfg.qk_nope_dim], rope_interleaved(q[..., cfg.qk_nope_dim:], pos, cfg.rope_theta)
        kv = x @ lw.wkv_a.t()
        self.ckv[i, start:end] = rms_norm(kv[:, :cfg.kv_lora_rank], lw.kv_norm, cfg.rms_norm_eps)
        self.kpe[i, start:end] = rope_interleaved(kv[:, cfg.kv_lora_rank:], pos, cfg.rope_theta)
        sel = self._indexer_select(lw, i, x, qin, pos, end)
        q_lat = torch.einsum("thn,hnc->thc", q_nope.float(), lw.w_uk.float())
        scores = torch.einsum("thc,sc->ths", q_lat, self.ckv[i, :end]) + torch.einsum("thr,sr->ths", q_pe, self.kpe[i, :end])
        scores = scores * cfg.qk_head_dim ** -0.5
        mask = torch.arange(end, device=x.device)[None, :] <= pos[:, None]              # causal [T, S]
        if sel is not None:
            keep = torch.zeros(t, end, dtype=torch.bool, device=x.device)
            keep.scatter_(1, sel, True)
            mask = mask & keep
        scores = scores.masked_fill(~mask[:, None, :], float("-inf"))
        p = scores.softmax(-1)
        o_lat = torch.einsum("ths,sc->thc", p, self.ckv[i, :end])
        o = torch.einsum("thc,hvc->thv", o_lat, lw.w_uv.float()).reshape(t, cfg.num_heads * cfg.v_head_dim)
        return o @ lw.wo.float().t()

    # ---- feed-forward
    def _ffn(self, lw: MlaLayer, x: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        if lw.dense is not None:
            return swiglu(x, *[m.float() for m in lw.dense])
        wts, idx = route(cfg, x, lw.gate_w, lw.gate_b)
        local = (idx >= self.w.expert_lo) & (idx < self.w.expert_hi)
        lidx = torch.where(local, idx - self.w.expert_lo, torch.full_like(idx, -1)).to(torch.int32)
        if cfg.expert_format == "fp4":
            w13, s13, w2, s2 = lw.experts
            y = cpu_moe_fp4(x.cpu(), lidx.cpu(), wts.cpu(), w13.cpu(), s13.cpu(), w2.cpu(), s2.cpu(),
                            cfg.expert_intermediate, cfg.swiglu_limit).to(x.device)
        else:
            w1, w3, w2 = lw.experts
            y = torch.zeros_like(x, dtype=torch.float32)
            for e in lidx.unique().tolist():
                if e < 0:
                    continue
                rows, ks = (lidx == e).nonzero(as_tuple=True)
                y.index_add_(0, rows, swiglu(x[rows].float(), w1[e].float(), w3[e].float(), w2[e].float(), cfg.swiglu_limit)
                             * wts[rows, ks, None])
        if self.comm is not None:
            y = self.comm.all_reduce(y)
        if lw.shared is not None:
            y = y + swiglu(x, *[m.float() for m in lw.shared])
        return y

    @torch.no_grad()
    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        """Append ``ids`` [T] to the context; returns fp32 logits [T, vocab]."""
        cfg, w = self.cfg, self.w
        t = ids.numel()
        if self.length + t > self.max_context:
            raise RuntimeError("sequence exceeds max_context")
        pos = torch.arange(self.length, self.length + t, device=self.device)
        h = w.embed[ids.long()].float()
        for i, lw in enumerate(w.layers):
            h = h + self._attention(lw, i, rms_norm(h, lw.attn_norm, cfg.rms_norm_eps), pos)
            h = h + self._ffn(lw, rms_norm(h, lw.ffn_norm, cfg.rms_norm_eps))
        self.length += t
        return rms_norm(h, w.norm, cfg.rms_norm_eps) @ w.head.float().t()

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new_tokens: int) -> tuple[list[int], torch.Tensor]:
        """Greedy decode; returns (tokens, fp32 logits of every generated position [n, vocab])."""
        self.reset()
        logits = self.forward(prompt.to(self.device))[-1:]
        toks, rows = [], []
        for _ in range(max_new_tokens):
            rows.append(logits[0])
            toks.append(int(logits[0].argmax()))
            if len(toks) == max_new_tokens:
                break
            logits = self.forward(torch.tensor([toks[-1]], device=self.device))
        return toks, torch.stack(rows)
