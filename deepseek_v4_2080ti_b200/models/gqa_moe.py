"""GQA + routed-expert family loaded from GGUF (MiniMax-M2.7-shaped): full-width QK RMSNorm, half-split partial RoPE,
sigmoid + bias top-k routing, SwiGLU experts stored as GGUF blocks that are decoded inside the tensor-core GEMM.

Parallel layout: attention heads are sharded over the tensor-parallel group (the reference replicates attention on every
rank, src/models/minimax_m2/architecture.py:85-267); routed experts are sharded by contiguous range (expert parallel)
and their weighted combine, the sum over ranks and the residual add run as one peer-memory kernel
(``PeerComm.moe_combine``); the output head is sharded over vocabulary rows with an arg-max merge.

Reference behaviour: src/models/minimax_m2/architecture.py (attention :213-267, route :291-298, MoE :300-385,
transformer :443-472), tensor names src/loader/mappings/minimax_m2.py:7-27, metadata keys src/models/minimax_m2/spec.py:36-60.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Iterator

import torch

from ..formats import gguf as G
from ..formats.gguf import GGMLType

ARCH = "minimax-m2"


@dataclass
class GqaMoeConfig:
    n_layers: int = 62
    hidden: int = 3072
    vocab: int = 200064
    n_heads: int = 48
    n_kv_heads: int = 8
    head_dim: int = 128
    rope_dim: int = 64
    rope_base: float = 5.0e6
    n_experts: int = 256
    top_k: int = 8
    moe_inter: int = 1536
    norm_eps: float = 1e-6
    context_length: int = 8192
    attn_type: str = "Q5_K"          # q / k / v / o projections
    dense_type: str = "Q4_K"         # embedding table and output head
    gate_up_type: str = "IQ1_M"      # routed w1 / w3
    down_type: str = "IQ2_XXS"       # routed w2

    @staticmethod
    def config3() -> "GqaMoeConfig":
        """The MiniMax-M2.7-shaped benchmark layout."""
        return GqaMoeConfig()

    @staticmethod
    def tiny(layers: int = 2, experts: int = 16, vocab: int = 512) -> "GqaMoeConfig":
        return GqaMoeConfig(n_layers=layers, hidden=512, vocab=vocab, n_heads=8, n_kv_heads=2, n_experts=experts, top_k=4,
                            moe_inter=256, context_length=512)

    def metadata(self) -> dict[str, Any]:
        a = ARCH
        return {"general.architecture": a, f"{a}.block_count": self.n_layers, f"{a}.embedding_length": self.hidden,
                f"{a}.vocab_size": self.vocab, f"{a}.context_length": self.context_length,
                f"{a}.attention.head_count": self.n_heads, f"{a}.attention.head_count_kv": self.n_kv_heads,
                f"{a}.attention.key_length": self.head_dim, f"{a}.rope.dimension_count": self.rope_dim,
                f"{a}.rope.freq_base": float(self.rope_base), f"{a}.expert_count": self.n_experts,
                f"{a}.expert_used_count": self.top_k, f"{a}.expert_feed_forward_length": self.moe_inter,
                f"{a}.expert_gating_func": 2, f"{a}.attention.layer_norm_rms_epsilon": float(self.norm_eps)}

    @staticmethod
    def from_metadata(md: dict[str, Any], tensors: dict | None = None) -> "GqaMoeConfig":
        a = str(md.get("general.architecture", ARCH))
        g = lambda k, d=0: md.get(f"{a}.{k}", d)
        cfg = GqaMoeConfig(n_layers=int(g("block_count")), hidden=int(g("embedding_length")), vocab=int(g("vocab_size")),
                           n_heads=int(g("attention.head_count")), n_kv_heads=int(g("attention.head_count_kv")),
                           head_dim=int(g("attention.key_length", 128)), rope_dim=int(g("rope.dimension_count", 64)),
                           rope_base=float(g("rope.freq_base", 1e4)), n_experts=int(g("expert_count")),
                           top_k=int(g("expert_used_count")), moe_inter=int(g("expert_feed_forward_length")),
                           norm_eps=float(g("attention.layer_norm_rms_epsilon", 1e-6)),
                           context_length=int(g("context_length", 8192)))
        if tensors:
            ty = lambda n, d: tensors[n].ggml_type.name if n in tensors else d
            cfg.attn_type, cfg.dense_type = ty("blk.0.attn_q.weight", cfg.attn_type), ty("output.weight", cfg.dense_type)
            cfg.gate_up_type = ty("blk.0.ffn_gate_exps.weight", cfg.gate_up_type)
            cfg.down_type = ty("blk.0.ffn_down_exps.weight", cfg.down_type)
        return cfg


def _q(w: torch.Tensor, tname: str) -> tuple[torch.Tensor, GGMLType]:
    t = GGMLType[tname]
    return G.quantize(w, t), t


def synth_tensors(cfg: GqaMoeConfig, seed: int = 0, device="cpu", std: float = 0.02, expert_pool: int | None = None
                  ) -> Iterator[tuple[str, torch.Tensor, GGMLType, tuple[int, ...]]]:
    """(gguf name, raw bytes, ggml type, logical shape) of a seeded random checkpoint in the reference's naming.
    ``expert_pool``: quantise only that many distinct experts per layer and repeat them (full-size benchmarks: the
    IQ quantisers search a codebook per group, which dominates start-up for 256 experts x 62 layers)."""
    # drawn on the target device (a 60-layer checkpoint is billions of values); every rank of a job uses the same
    # device type and seed, so all ranks see the same tensors
    gdev = torch.device(device)
    gen = torch.Generator(device=gdev).manual_seed(seed)
    rnd = lambda *s, sd=std: torch.randn(*s, generator=gen, device=gdev) * sd
    f32 = lambda w: (w.float().contiguous().view(torch.uint8), GGMLType.F32)
    h, d = cfg.hidden, cfg.head_dim
    qd, kvd = cfg.n_heads * d, cfg.n_kv_heads * d
    yield ("token_embd.weight", *_q(rnd(cfg.vocab, h), cfg.dense_type), (cfg.vocab, h))
    yield ("output.weight", *_q(rnd(cfg.vocab, h), cfg.dense_type), (cfg.vocab, h))
    yield ("output_norm.weight", *f32(1.0 + rnd(h, sd=0.1)), (h,))
    for i in range(cfg.n_layers):
        p = f"blk.{i}."
        yield (p + "attn_norm.weight", *f32(1.0 + rnd(h, sd=0.1)), (h,))
        yield (p + "ffn_norm.weight", *f32(1.0 + rnd(h, sd=0.1)), (h,))
        yield (p + "attn_q.weight", *_q(rnd(qd, h), cfg.attn_type), (qd, h))
        yield (p + "attn_k.weight", *_q(rnd(kvd, h), cfg.attn_type), (kvd, h))
        yield (p + "attn_v.weight", *_q(rnd(kvd, h), cfg.attn_type), (kvd, h))
        yield (p + "attn_output.weight", *_q(rnd(h, qd), cfg.attn_type), (h, qd))
        yield (p + "attn_q_norm.weight", *f32(1.0 + rnd(qd, sd=0.1)), (qd,))
        yield (p + "attn_k_norm.weight", *f32(1.0 + rnd(kvd, sd=0.1)), (kvd,))
        yield (p + "ffn_gate_inp.weight", *f32(rnd(cfg.n_experts, h, sd=0.05)), (cfg.n_experts, h))
        yield (p + "exp_probs_b.bias", *f32(rnd(cfg.n_experts, sd=0.02)), (cfg.n_experts,))
        pool = min(cfg.n_experts, expert_pool or cfg.n_experts)
        reps = (cfg.n_experts + pool - 1) // pool
        for name, shape, tname in (("ffn_gate_exps", (cfg.moe_inter, h), cfg.gate_up_type),
                                   ("ffn_up_exps", (cfg.moe_inter, h), cfg.gate_up_type),
                                   ("ffn_down_exps", (h, cfg.moe_inter), cfg.down_type)):
            raw, t = _q(rnd(pool * shape[0], shape[1]), tname)
            raw = raw.view(pool, shape[0], -1).repeat(reps, 1, 1)[:cfg.n_experts].contiguous()
            yield (p + name + ".weight", raw, t, (cfg.n_experts, *shape))


def write_synthetic_gguf(path: str, cfg: GqaMoeConfig, seed: int = 0, std: float = 0.02, expert_pool: int | None = None) -> None:
    G.write_gguf(path, cfg.metadata(), synth_tensors(cfg, seed, "cpu", std, expert_pool))


# ---------------------------------------------------------------------------------------------- fp32 oracle
def _rope_half(x: torch.Tensor, pos: torch.Tensor, rope_dim: int, base: float) -> torch.Tensor:
    half = rope_dim // 2
    inv = base ** (-(2.0 * torch.arange(half, dtype=torch.float64)) / rope_dim)
    ang = pos.double()[:, None] * inv[None, :]
    cos, sin = ang.cos().float()[:, None, :], ang.sin().float()[:, None, :]
    a, b = x[..., :half], x[..., half:rope_dim]
    return torch.cat([a * cos - b * sin, a * sin + b * cos, x[..., rope_dim:]], -1)


class GqaMoeReference:
    """Plain fp32 PyTorch model over the dequantised tensors of a bundle (CPU oracle for tokens and logits)."""

    def __init__(self, cfg: GqaMoeConfig, tensors: dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, {k: v.float() for k, v in tensors.items()}
        self.k = [torch.zeros(0, cfg.n_kv_heads, cfg.head_dim) for _ in range(cfg.n_layers)]
        self.v = [torch.zeros(0, cfg.n_kv_heads, cfg.head_dim) for _ in range(cfg.n_layers)]

    @staticmethod
    def _norm(x, g, eps):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * g

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        """Appends ``ids`` to the context; returns fp32 logits [T, vocab]."""
        cfg, w = self.cfg, self.w
        t = ids.numel()
        start = self.k[0].shape[0]
        pos = torch.arange(start, start + t)
        x = w["token_embd.weight"][ids.long()]
        for i in range(cfg.n_layers):
            p = f"blk.{i}."
            xn = self._norm(x, w[p + "attn_norm.weight"], cfg.norm_eps)
            q = self._norm(xn @ w[p + "attn_q.weight"].t(), w[p + "attn_q_norm.weight"], cfg.norm_eps)
            k = self._norm(xn @ w[p + "attn_k.weight"].t(), w[p + "attn_k_norm.weight"], cfg.norm_eps)
            v = xn @ w[p + "attn_v.weight"].t()
            q = _rope_half(q.view(t, cfg.n_heads, cfg.head_dim), pos, cfg.rope_dim, cfg.rope_base)
            k = _rope_half(k.view(t, cfg.n_kv_heads, cfg.head_dim), pos, cfg.rope_dim, cfg.rope_base)
            self.k[i] = torch.cat([self.k[i], k])
            self.v[i] = torch.cat([self.v[i], v.view(t, cfg.n_kv_heads, cfg.head_dim)])
            rep = cfg.n_heads // cfg.n_kv_heads
            kk, vv = self.k[i].repeat_interleave(rep, 1), self.v[i].repeat_interleave(rep, 1)
            s = torch.einsum("thd,shd->hts", q, kk) / math.sqrt(cfg.head_dim)
            mask = torch.arange(start + t)[None, :] > pos[:, None]
            s = s.masked_fill(mask[None], float("-inf")).softmax(-1)
            o = torch.einsum("hts,shd->thd", s, vv).reshape(t, -1)
            x = x + o @ w[p + "attn_output.weight"].t()
            xn = self._norm(x, w[p + "ffn_norm.weight"], cfg.norm_eps)
            probs = torch.sigmoid(xn @ w[p + "ffn_gate_inp.weight"].t())
            _, idx = torch.topk(probs + w[p + "exp_probs_b.bias"], cfg.top_k, -1)
            wt = torch.gather(probs, -1, idx)
            wt = wt / wt.sum(-1, keepdim=True).clamp_min(1e-20)
            y = torch.zeros_like(x)
            for e in idx.unique().tolist():
                tok, slot = (idx == e).nonzero(as_tuple=True)
                xe = xn[tok]
                a = torch.nn.functional.silu(xe @ w[p + "ffn_gate_exps.weight"][e].t()) * (xe @ w[p + "ffn_up_exps.weight"][e].t())
                y.index_add_(0, tok, (a @ w[p + "ffn_down_exps.weight"][e].t()) * wt[tok, slot][:, None])
            x = x + y
        x = self._norm(x, w["output_norm.weight"], cfg.norm_eps)
        return x @ w["output.weight"].t()

    def generate(self, prompt: torch.Tensor, n: int) -> list[int]:
        out = [int(self.forward(prompt)[-1].argmax())]
        while len(out) < n:
            out.append(int(self.forward(torch.tensor([out[-1]]))[-1].argmax()))
        return out


# ---------------------------------------------------------------------------------------------- GPU runtime
class TensorStore:
    """Uniform access to raw GGUF tensors, from a bundle on disk or from an in-memory iterator of
    ``(name, raw, type, shape)`` (synthetic benchmarks skip the file)."""

    def __init__(self, src):
        if hasattr(src, "tensors") and hasattr(src, "raw"):
            self._b, self._d = src, None
        else:
            self._b, self._d = None, {n: (raw, GGMLType(t), tuple(shape)) for n, raw, t, shape in src}

    def get(self, name: str) -> tuple[torch.Tensor, GGMLType, tuple[int, ...]]:
        """raw uint8 [..., rows, row_bytes], type, logical shape."""
        if self._d is not None:
            raw, t, shape = self._d[name]
            if t == GGMLType.F32:
                return raw, t, shape
            return raw.reshape(*shape[:-1], -1), t, shape
        ti = self._b.tensors[name]
        return self._b.raw(name), ti.ggml_type, tuple(ti.shape)

    def names(self) -> list[str]:
        return list(self._d) if self._d is not None else list(self._b.tensors)

    def dequantized(self) -> dict[str, torch.Tensor]:
        """Every tensor as fp32 in its logical shape (input of the fp32 oracle)."""
        out = {}
        for n in self.names():
            raw, t, shape = self.get(n)
            out[n] = self.f32(n) if t == GGMLType.F32 else \
                G.dequantize(raw.reshape(-1, raw.shape[-1]).clone(), t, shape[-1]).reshape(shape)
        return out

    def f32(self, name: str) -> torch.Tensor:
        raw, t, shape = self.get(name)
        assert t == GGMLType.F32, (name, t)
        return raw.contiguous().reshape(-1).view(torch.float32).reshape(shape).clone()


@dataclass
class GqaMoeLayer:
    attn_norm: torch.Tensor
    ffn_norm: torch.Tensor
    qkv: Any                      # GGUFLinear, rows [q heads | k heads | v heads] of this rank
    o: Any                        # GGUFLinear over this rank's slice of the attention width
    q_gamma: torch.Tensor
    k_gamma: torch.Tensor
    gate: Any                     # PackedLinear bf16 [E, H]
    gate_bias: torch.Tensor
    w13: Any
    w2: Any


class GqaMoeGpuWeights:
    def __init__(self, cfg: GqaMoeConfig, src, device="cuda", rank: int = 0, world: int = 1):
        from ..ops import gguf_gemm, moe
        from ..ops.gemm import PackedLinear
        self.cfg, self.device, self.rank, self.world = cfg, torch.device(device), rank, world
        assert cfg.n_heads % world == 0 and cfg.n_kv_heads % world == 0 and cfg.n_experts % world == 0
        assert cfg.head_dim == 128
        st = src if isinstance(src, TensorStore) else TensorStore(src)
        dev, d = self.device, cfg.head_dim
        self.hq, self.hkv = cfg.n_heads // world, cfg.n_kv_heads // world
        per = cfg.n_experts // world
        self.expert_lo = rank * per
        bf = lambda x: x.to(dev, torch.bfloat16).contiguous()

        def rows(name, lo, hi):
            raw, t, shape = st.get(name)
            return raw[lo:hi], t, shape

        raw, t, shape = st.get("token_embd.weight")
        self.embed = bf(G.dequantize(raw.to(dev).reshape(shape[0], -1), t, shape[1]))
        self.final_norm = bf(st.f32("output_norm.weight"))
        n = (cfg.vocab + world - 1) // world
        self.head_lo, hi = rank * n, min(cfg.vocab, (rank + 1) * n)
        raw, t, shape = rows("output.weight", self.head_lo, hi)
        self.head = gguf_gemm.GGUFLinear.from_raw(raw, t, hi - self.head_lo, shape[1], dev)
        self.layers: list[GqaMoeLayer] = []
        for i in range(cfg.n_layers):
            p = f"blk.{i}."
            q, t, shape = rows(p + "attn_q.weight", rank * self.hq * d, (rank + 1) * self.hq * d)
            k, _, _ = rows(p + "attn_k.weight", rank * self.hkv * d, (rank + 1) * self.hkv * d)
            v, _, _ = rows(p + "attn_v.weight", rank * self.hkv * d, (rank + 1) * self.hkv * d)
            qkv = gguf_gemm.GGUFLinear.from_raw(torch.cat([q, k, v]), t, (self.hq + 2 * self.hkv) * d, cfg.hidden, dev)
            raw, t, shape = st.get(p + "attn_output.weight")
            be, bb = G.BLOCK_ELEMS[t], G.BLOCK_BYTES[t]
            kl = self.hq * d
            assert kl % be == 0, "attention width per rank must hold whole quantisation blocks"
            o_raw = raw.reshape(shape[0], shape[1] // be, bb)[:, rank * kl // be:(rank + 1) * kl // be].reshape(shape[0], -1)
            o = gguf_gemm.GGUFLinear.from_raw(o_raw.contiguous(), t, shape[0], kl, dev)
            qg = st.f32(p + "attn_q_norm.weight")[rank * self.hq * d:(rank + 1) * self.hq * d]
            kg = st.f32(p + "attn_k_norm.weight")[rank * self.hkv * d:(rank + 1) * self.hkv * d]
            w1, t1, s1 = st.get(p + "ffn_gate_exps.weight")
            w3, _, _ = st.get(p + "ffn_up_exps.weight")
            w2, t2, s2 = st.get(p + "ffn_down_exps.weight")
            lo, hi_e = self.expert_lo, self.expert_lo + per
            w13 = moe.ExpertWeights.from_gguf([torch.cat([w1[e], w3[e]]).to(dev) for e in range(lo, hi_e)], t1,
                                              2 * cfg.moe_inter, cfg.hidden)
            w2e = moe.ExpertWeights.from_gguf([w2[e].to(dev) for e in range(lo, hi_e)], t2, cfg.hidden, cfg.moe_inter)
            self.layers.append(GqaMoeLayer(
                bf(st.f32(p + "attn_norm.weight")), bf(st.f32(p + "ffn_norm.weight")), qkv, o, bf(qg), bf(kg),
                PackedLinear.from_bf16(bf(st.f32(p + "ffn_gate_inp.weight"))),
                st.f32(p + "exp_probs_b.bias").to(dev).contiguous(), w13, w2e))

    def nbytes(self) -> int:
        n = self.embed.numel() * 2 + self.head.nbytes()
        for l in self.layers:
            n += l.qkv.nbytes() + l.o.nbytes() + l.w13.weight.numel() + l.w2.weight.numel() + l.gate.nbytes()
        return n


class _NoComm:
    world, rank = 1, 0

    def all_reduce(self, t):
        return t

    def argmax_merge(self, idx, val):
        return idx


@dataclass
class _Seq:
    slot: int
    blocks: list[int] = field(default_factory=list)
    length: int = 0


class GqaMoeRuntime:
    """Paged-KV runtime: chunked prefill of one sequence, batched decode (CUDA-graph replay per batch size)."""

    def __init__(self, cfg: GqaMoeConfig, weights: GqaMoeGpuWeights, max_slots: int = 1, max_context: int = 4096 + 512,
                 block_size: int = 64, comm=None):
        from ..ops import attention
        self.cfg, self.w, self.device = cfg, weights, weights.device
        self.comm = comm or _NoComm()
        assert self.comm.world == weights.world
        self.block_size, self.max_slots = block_size, max_slots
        self.max_blocks = (max_context + block_size - 1) // block_size
        self.num_blocks = self.max_blocks * max_slots + 1
        dev = self.device
        self.k_cache = torch.zeros(cfg.n_layers, self.num_blocks, weights.hkv, block_size, 128, dtype=torch.bfloat16, device=dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.inv_freq = attention.rope_inv_freq(cfg.rope_dim, cfg.rope_base, dev)
        self.free_blocks = list(range(self.num_blocks - 1, 0, -1))
        self.free_slots = list(range(max_slots - 1, -1, -1))
        self.seqs: dict[int, _Seq] = {}
        self.block_table = torch.zeros(max_slots, self.max_blocks, dtype=torch.int32, device=dev)
        self._bt_host = torch.zeros(max_slots, self.max_blocks, dtype=torch.int32)
        self._graphs: dict[tuple, dict] = {}
        self.launches = 0

    def allocate(self) -> int:
        s = self.free_slots.pop()
        self.seqs[s] = _Seq(s)
        return s

    def free(self, slot: int) -> None:
        st = self.seqs.pop(slot)
        self.free_blocks.extend(reversed(st.blocks))
        self.free_slots.append(slot)

    def _ensure(self, st: _Seq, new_len: int) -> None:
        need = (new_len + self.block_size - 1) // self.block_size
        if need > self.max_blocks:
            raise RuntimeError("sequence exceeds max_context")
        grown = False
        while len(st.blocks) < need:
            if not self.free_blocks:
                raise RuntimeError("KV cache exhausted")
            b = self.free_blocks.pop()
            self._bt_host[st.slot, len(st.blocks)] = b
            st.blocks.append(b)
            grown = True
        if grown:
            self.block_table[st.slot].copy_(self._bt_host[st.slot], non_blocking=True)

    # ---- one forward pass over T rows
    def _forward(self, ids, positions, kv_slots, meta, last_rows: torch.Tensor | None) -> torch.Tensor:
        from ..ops import attention, basic, gemm, gguf_gemm, moe
        cfg, w, comm = self.cfg, self.w, self.comm
        t = ids.numel()
        d = 128
        qw, kw = w.hq * d, w.hkv * d
        h = basic.embedding(ids, w.embed, 0, cfg.vocab)
        delta = None
        for i, L in enumerate(w.layers):
            x = basic.rmsnorm(h, L.attn_norm, cfg.norm_eps, False) if delta is None else \
                basic.add_rmsnorm(h, delta, L.attn_norm, cfg.norm_eps, False)
            proj = gguf_gemm.linear(x, L.qkv)
            ss = attention.qk_sumsq(proj, 0, qw, qw, kw)
            if comm.world > 1:
                ss = comm.all_reduce(ss)
            q = attention.qk_fullnorm_rope_append(proj, 0, qw, qw + kw, L.q_gamma, L.k_gamma, ss, cfg.n_heads * d,
                                                  cfg.n_kv_heads * d, cfg.norm_eps, self.inv_freq, cfg.rope_dim, positions,
                                                  kv_slots, self.k_cache[i], self.v_cache[i], w.hq, w.hkv)
            if meta["mode"] == "prefill":
                o = attention.prefill(q, self.k_cache[i], self.v_cache[i], meta["block_table"], meta["q_start"],
                                      meta["q_len"], meta["kv_len"], meta["max_q_len"])
            else:
                o = attention.decode(q, self.k_cache[i], self.v_cache[i], meta["block_table"], meta["kv_len"],
                                     max_kv_len=meta["max_kv_len"])
            d_attn = comm.all_reduce(gguf_gemm.linear(o.view(t, qw), L.o))
            xn = basic.add_rmsnorm(h, d_attn, L.ffn_norm, cfg.norm_eps, False)      # h += d_attn
            logits = gemm.linear(xn, L.gate, out_f32=True)
            idx, wts = moe.route(logits, L.gate_bias, cfg.top_k, "sigmoid", True, 1.0)
            # combine + sum over the expert-parallel ranks + residual in one kernel; the result is the new stream
            h = moe.experts_forward(xn, idx, wts, L.w13, L.w2, w.expert_lo, comm=comm if comm.world > 1 else None,
                                    residual=h)
            delta = None
        if last_rows is not None:
            h = h.index_select(0, last_rows)
        x = basic.rmsnorm(h, w.final_norm, cfg.norm_eps, False)
        return gguf_gemm.linear(x, w.head, out_f32=True)

    def _next(self, logits: torch.Tensor) -> torch.Tensor:
        from ..ops import basic
        idx, val = basic.argmax(logits, self.w.head_lo, True)
        return self.comm.argmax_merge(idx, val)

    @torch.no_grad()
    def prefill(self, slot: int, token_ids: torch.Tensor, chunk: int = 4096) -> torch.Tensor:
        from ..ops import _lib
        st = self.seqs[slot]
        l0 = _lib.LAUNCHES
        nxt, total, dev = None, token_ids.numel(), self.device
        i32 = lambda v: torch.tensor([v], dtype=torch.int32, device=dev)
        for s in range(0, total, chunk):
            ids = token_ids[s:s + chunk]
            t = ids.numel()
            self._ensure(st, st.length + t)
            pos = torch.arange(st.length, st.length + t, dtype=torch.int32, device=dev)
            row = self.block_table[slot]
            kv_slots = (row[(pos // self.block_size).long()] * self.block_size + pos % self.block_size).to(torch.int32)
            meta = {"mode": "prefill", "block_table": self.block_table[slot:slot + 1], "q_start": i32(0), "q_len": i32(t),
                    "kv_len": i32(st.length + t), "max_q_len": t}
            logits = self._forward(ids, pos, kv_slots, meta, torch.tensor([t - 1], dtype=torch.int64, device=dev))
            st.length += t
            if s + t >= total:
                nxt = self._next(logits)
        self.launches = _lib.LAUNCHES - l0
        return nxt

    def _decode_body(self, buf, bucket: int) -> torch.Tensor:
        meta = {"mode": "decode", "block_table": buf["bt"], "kv_len": buf["kv_len"], "max_kv_len": bucket}
        return self._next(self._forward(buf["ids"], buf["pos"], buf["kv_slots"], meta, None))

    @torch.no_grad()
    def decode(self, slots: list[int], token_ids: torch.Tensor, use_graph: bool = True) -> torch.Tensor:
        from ..ops import _lib
        b, dev = len(slots), self.device
        sts = [self.seqs[s] for s in slots]
        for st in sts:
            self._ensure(st, st.length + 1)
        bucket = 1 << max(10, max(st.length for st in sts).bit_length())
        entry = self._graphs.setdefault((b, bucket), {"buf": None, "graph": None})
        if entry["buf"] is None:
            z = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
            entry["buf"] = {"ids": z(b), "pos": z(b), "kv_slots": z(b), "kv_len": z(b) + 1, "bt": z(b, self.max_blocks)}
        buf = entry["buf"]
        host = torch.tensor([[st.length, st.length + 1, st.slot,
                              st.blocks[st.length // self.block_size] * self.block_size + st.length % self.block_size]
                             for st in sts], dtype=torch.int32).to(dev, non_blocking=True)
        buf["ids"].copy_(token_ids)
        buf["pos"].copy_(host[:, 0])
        buf["kv_len"].copy_(host[:, 1])
        buf["kv_slots"].copy_(host[:, 3])
        buf["bt"].copy_(self.block_table[host[:, 2].long()])
        if not use_graph:
            l0 = _lib.LAUNCHES
            out = self._decode_body(buf, bucket)
            self.launches = _lib.LAUNCHES - l0
        else:
            if entry["graph"] is None:
                self._decode_body(buf, bucket)          # warm-up: the K/V row written here is rewritten by the replay
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                l0 = _lib.LAUNCHES
                with torch.cuda.graph(g):
                    entry["out"] = self._decode_body(buf, bucket)
                entry["graph"], entry["launches"] = g, _lib.LAUNCHES - l0
            entry["graph"].replay()
            self.launches = entry["launches"]
            out = entry["out"]
        for st in sts:
            st.length += 1
        return out

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new_tokens: int, chunk: int = 4096, use_graph: bool = True) -> list[int]:
        slot = self.allocate()
        try:
            tok = self.prefill(slot, prompt.to(self.device, torch.int32), chunk)
            out = [int(tok.item())]
            while len(out) < max_new_tokens:
                tok = self.decode([slot], tok.to(torch.int32), use_graph)
                out.append(int(tok.item()))
            return out
        finally:
            self.free(slot)
