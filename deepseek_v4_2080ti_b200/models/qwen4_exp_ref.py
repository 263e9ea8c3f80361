"""Qwen4-Exp-style decoder (hyper-connection streams, Gated DeltaNet and QSA sparse-attention layers, routed experts
with a gated shared expert, hashed n-gram "PLE" injection) assembled from this package's components as an fp32 CPU
runtime with caches: the executable statement of that family's forward pass for tiny configurations, and the oracle a
GPU runtime of the family would be checked against.  Not a served shape on the GPU path.

Layer (reference: src/models/qwen4_exp/model.py:137-289):  streams [B, S, hc * H]
    (+ PLE(streams, token history) on the layers that have one                      model.py:56-134)
    mixed, inject = gated_residual(streams)           -> attention (Gated DeltaNet | QSA) -> inject into streams
    mixed, inject = gated_residual(streams)           -> router top-k experts + sigmoid-gated shared expert -> inject
Model (model.py:312-421): embed, repeat into hc streams, layers, final gated mixer (no injection), lm_head.
Gated DeltaNet mixer: attention.py:312-436; QSA attention and its block-pooled indexer: attention.py:461-737.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from ..ops.gdn import recurrent_ref
from . import qwen4_exp_components as C


@dataclass
class Qwen4ExpConfig:
    vocab_size: int = 300
    hidden_size: int = 64
    num_layers: int = 4
    full_attention_interval: int = 2            # layers i with (i + 1) % interval == 0 are QSA attention layers
    hc_count: int = 4
    hc_rank: int = 16                           # width of the hyper-connection mixer's bottleneck
    rms_norm_eps: float = 1e-6
    # QSA attention
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 32
    rope_theta: float = 10000.0
    mrope_sections: tuple[int, int, int] = (8, 4, 4)
    indexer_heads: int = 2
    indexer_head_dim: int = 32
    indexer_budget: int = 16
    indexer_compress_ratio: int = 4
    # Gated DeltaNet (the recurrence oracle is written for 128-wide heads)
    linear_k_heads: int = 1
    linear_v_heads: int = 2
    linear_head_dim: int = 128
    conv_kernel: int = 4
    # feed-forward
    num_experts: int = 4
    experts_per_token: int = 2
    moe_intermediate: int = 32
    shared_intermediate: int = 32
    norm_topk: bool = True
    # hashed n-gram injection
    ple_layers: tuple[int, ...] = (1,)
    ngram_size: int = 3
    heads_per_ngram: int = 2
    ngram_head_vocab: tuple[int, ...] = (31, 37, 41, 43)       # (ngram_size - 1) * heads_per_ngram prime table sizes
    ngram_embed_dim: int = 8
    ple_conv_kernel: int = 2
    ngram_seed: int = 1234
    eos_token_id: int = 0
    layer_types: list[str] = field(default_factory=list)

    def __post_init__(self):
        if not self.layer_types:
            self.layer_types = ["full" if (i + 1) % self.full_attention_interval == 0 else "linear" for i in range(self.num_layers)]
        assert len(self.ngram_head_vocab) == (self.ngram_size - 1) * self.heads_per_ngram
        assert self.linear_head_dim == 128 and self.linear_v_heads % self.linear_k_heads == 0


def synth_weights(cfg: Qwen4ExpConfig, seed: int = 0, std: float = 0.05) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, sd=std: torch.randn(*s, generator=g) * sd
    one = lambda *s: 1.0 + r(*s, sd=0.05)
    h, hc = cfg.hidden_size, cfg.hc_count
    w = {"embed": r(cfg.vocab_size, h, sd=0.5), "lm_head": r(cfg.vocab_size, h),
         "final.hc_norm": one(hc * h), "final.down": r(cfg.hc_rank, hc * h), "final.up": r(hc * h, cfg.hc_rank)}
    kd, vd = cfg.linear_k_heads * 128, cfg.linear_v_heads * 128
    for i, lt in enumerate(cfg.layer_types):
        p = f"layers.{i}."
        for blk in ("attn_hc", "mlp_hc"):
            w[p + blk + ".hc_norm"], w[p + blk + ".down"] = one(hc * h), r(cfg.hc_rank, hc * h)
            w[p + blk + ".up"], w[p + blk + ".inject"] = r(hc * h, cfg.hc_rank), r(hc, hc * h)
        if lt == "linear":
            a = p + "linear_attn."
            w[a + "in_proj_qkv"], w[a + "in_proj_z"] = r(2 * kd + vd, h), r(vd, h)
            w[a + "in_proj_a"], w[a + "in_proj_b"] = r(cfg.linear_v_heads, h), r(cfg.linear_v_heads, h)
            w[a + "conv1d"] = r(2 * kd + vd, cfg.conv_kernel, sd=0.3)
            w[a + "A_log"], w[a + "dt_bias"] = r(cfg.linear_v_heads, sd=0.3), r(cfg.linear_v_heads, sd=0.3)
            w[a + "norm"], w[a + "out_proj"] = one(128), r(h, vd)
        else:
            a = p + "self_attn."
            d = cfg.head_dim
            w[a + "q_proj"], w[a + "k_proj"] = r(cfg.num_heads * d * 2, h), r(cfg.num_kv_heads * d, h)
            w[a + "v_proj"], w[a + "o_proj"] = r(cfg.num_kv_heads * d, h), r(h, cfg.num_heads * d)
            w[a + "q_norm"], w[a + "k_norm"] = one(d), one(d)
            di = cfg.indexer_head_dim
            w[a + "index_qk_proj"] = r((cfg.indexer_heads + 1) * di, h, sd=0.2)
            w[a + "q_layernorm"], w[a + "k_layernorm"] = one(di), one(di)
        m = p + "mlp."
        w[m + "gate"] = r(cfg.num_experts, h, sd=0.3)
        for e in range(cfg.num_experts):
            w[m + f"experts.{e}.gate_proj"], w[m + f"experts.{e}.up_proj"] = r(cfg.moe_intermediate, h), r(cfg.moe_intermediate, h)
            w[m + f"experts.{e}.down_proj"] = r(h, cfg.moe_intermediate)
        w[m + "shared.gate_proj"], w[m + "shared.up_proj"] = r(cfg.shared_intermediate, h), r(cfg.shared_intermediate, h)
        w[m + "shared.down_proj"], w[m + "shared_gate"] = r(h, cfg.shared_intermediate), r(1, h)
        if i in cfg.ple_layers:
            q = p + "ple."
            e_in = len(cfg.ngram_head_vocab) * cfg.ngram_embed_dim
            w[q + "table"] = r(sum(cfg.ngram_head_vocab), cfg.ngram_embed_dim, sd=0.5)
            w[q + "key_proj"], w[q + "value_proj"] = r(hc * h, e_in, sd=0.2), r(h, e_in, sd=0.2)
            w[q + "norm_key"], w[q + "norm_query"], w[q + "norm_conv"] = one(hc * h), one(hc * h), one(hc * h)
            w[q + "conv1d"] = r(hc * h, cfg.ple_conv_kernel, sd=0.3)
    return w


def _rms(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()


def _swiglu(x, gate, up, down):
    return F.linear(F.silu(F.linear(x, gate)) * F.linear(x, up), down)


class Qwen4ExpRef:
    """One sequence, fp32, CPU.  ``forward(ids)`` appends ``ids`` to the context and returns logits [T, vocab]."""

    def __init__(self, cfg: Qwen4ExpConfig, weights: dict[str, torch.Tensor], max_context: int = 512):
        self.cfg, self.w, self.max_context = cfg, {k: v.float() for k, v in weights.items()}, max_context
        self.rot = 2 * sum(cfg.mrope_sections)
        assert self.rot <= cfg.head_dim and self.rot <= cfg.indexer_head_dim
        pos = torch.arange(max_context).view(1, -1)
        self.cos, self.sin = C.mrope_cos_sin(pos, self.rot, cfg.rope_theta, cfg.mrope_sections)   # [1, ctx, rot]
        sizes = torch.tensor(cfg.ngram_head_vocab, dtype=torch.long)
        self._sizes, self._offsets = sizes, torch.cumsum(sizes, 0) - sizes
        self._mult = {i: C.ngram_multipliers(cfg.vocab_size, cfg.ngram_size, j, cfg.ngram_seed)
                      for j, i in enumerate(cfg.ple_layers)}
        self.reset()

    def reset(self) -> None:
        cfg = self.cfg
        self.length = 0
        self.history = torch.full((1, cfg.ngram_size - 1), cfg.eos_token_id, dtype=torch.long)
        self.cache: list[dict] = []
        for lt in cfg.layer_types:
            if lt == "linear":
                cdim = 2 * cfg.linear_k_heads * 128 + cfg.linear_v_heads * 128
                self.cache.append({"conv": torch.zeros(cdim, cfg.conv_kernel - 1),
                                   "state": torch.zeros(cfg.linear_v_heads, 128, 128)})
            else:
                self.cache.append({"k": torch.zeros(0, cfg.num_kv_heads, cfg.head_dim), "v": torch.zeros(0, cfg.num_kv_heads, cfg.head_dim),
                                   "index_k": torch.zeros(0, cfg.indexer_head_dim)})
        self.ple_conv = {i: torch.zeros(cfg.hc_count * cfg.hidden_size, (cfg.ple_conv_kernel - 1) * cfg.ngram_size)
                         for i in cfg.ple_layers}

    def snapshot(self) -> dict:
        """Copy of every cache (recurrent state, convolution tails, KV, token history): what a speculative verify pass
        saves so that a rejected block can be undone."""
        return copy.deepcopy({"length": self.length, "history": self.history, "cache": self.cache, "ple_conv": self.ple_conv})

    def restore(self, snap: dict) -> None:
        snap = copy.deepcopy(snap)
        self.length, self.history, self.cache, self.ple_conv = snap["length"], snap["history"], snap["cache"], snap["ple_conv"]

    # ---- pieces
    def _ple(self, i: int, streams: torch.Tensor, history: torch.Tensor) -> torch.Tensor:
        cfg, w, p = self.cfg, self.w, f"layers.{i}.ple."
        s, h, hc = streams.shape[0], cfg.hidden_size, cfg.hc_count
        rows = C.ngram_row_ids(history, s, cfg.ngram_size, cfg.heads_per_ngram, self._sizes, self._offsets, self._mult[i],
                               cfg.eos_token_id)[0]                                      # [S, heads]
        emb = w[p + "table"][rows].flatten(-2)                                           # [S, heads * embed]
        key = C._group_rms(F.linear(emb, w[p + "key_proj"]), w[p + "norm_key"], h, cfg.rms_norm_eps).unflatten(-1, (hc, h))
        value = F.linear(emb, w[p + "value_proj"])
        query = C._group_rms(streams, w[p + "norm_query"], h, cfg.rms_norm_eps).unflatten(-1, (hc, h))
        gate = (key * query).sum(-1, keepdim=True) / math.sqrt(h)
        gate = gate.abs().clamp_min(1e-6).sqrt() * gate.sign()                           # signed square root
        gated = (torch.sigmoid(gate) * value.unsqueeze(-2)).flatten(-2)                  # [S, hc * H]
        normed = C._group_rms(gated, w[p + "norm_conv"], h, cfg.rms_norm_eps)
        # dilated depthwise causal convolution over the sequence (dilation = n-gram size), then SiLU
        x = torch.cat([self.ple_conv[i], normed.t()], -1)                                # [C, state + S]
        self.ple_conv[i] = x[:, -self.ple_conv[i].shape[1]:].clone() if self.ple_conv[i].shape[1] else self.ple_conv[i]
        conv = F.conv1d(x[None], w[p + "conv1d"][:, None, :], None, dilation=cfg.ngram_size, groups=x.shape[0])[0]
        return gated + F.silu(conv[:, -s:]).t()

    def _deltanet(self, i: int, x: torch.Tensor) -> torch.Tensor:
        cfg, w, p, c = self.cfg, self.w, f"layers.{i}.linear_attn.", self.cache[i]
        s = x.shape[0]
        kd, vd = cfg.linear_k_heads * 128, cfg.linear_v_heads * 128
        mixed = torch.cat([c["conv"], F.linear(x, w[p + "in_proj_qkv"]).t()], -1)        # [C, k - 1 + S]
        c["conv"] = mixed[:, -(cfg.conv_kernel - 1):].clone()
        mixed = F.silu(F.conv1d(mixed[None], w[p + "conv1d"][:, None, :], None, groups=mixed.shape[0])[0][:, -s:]).t()
        q, k, v = mixed.split([kd, kd, vd], -1)
        beta = torch.sigmoid(F.linear(x, w[p + "in_proj_b"]))
        g = -w[p + "A_log"].exp() * F.softplus(F.linear(x, w[p + "in_proj_a"]) + w[p + "dt_bias"])
        o, c["state"] = recurrent_ref(q.reshape(s, -1, 128), k.reshape(s, -1, 128), v.reshape(s, -1, 128), g, beta, c["state"])
        z = F.linear(x, w[p + "in_proj_z"]).view(s, -1, 128)
        o = _rms(o, w[p + "norm"], cfg.rms_norm_eps) * F.silu(z)
        return F.linear(o.reshape(s, vd), w[p + "out_proj"])

    def _qsa(self, i: int, x: torch.Tensor, past: int) -> torch.Tensor:
        cfg, w, p, c = self.cfg, self.w, f"layers.{i}.self_attn.", self.cache[i]
        s, d, di = x.shape[0], cfg.head_dim, cfg.indexer_head_dim
        end = past + s
        cos, sin = self.cos[:, past:end], self.sin[:, past:end]
        qk = F.linear(x, w[p + "index_qk_proj"])
        qi = _rms(qk[:, :cfg.indexer_heads * di].view(s, -1, di), w[p + "q_layernorm"], cfg.rms_norm_eps)
        qi = C.apply_rotary_half(qi[None], cos, sin)                                       # [1, S, Hi, di]
        c["index_k"] = torch.cat([c["index_k"], qk[:, cfg.indexer_heads * di:]])
        sel = C.qsa_select(qi, c["index_k"][None], w[p + "k_layernorm"], self.cos[:, :end], self.sin[:, :end], past,
                           cfg.indexer_budget, cfg.indexer_compress_ratio, cfg.rms_norm_eps)[0]        # [S, width]
        qg = F.linear(x, w[p + "q_proj"]).view(s, cfg.num_heads, 2 * d)
        q, gate = qg[..., :d], qg[..., d:].reshape(s, -1)
        q = C.apply_rotary_half(_rms(q, w[p + "q_norm"], cfg.rms_norm_eps)[None], cos, sin)[0]
        k = C.apply_rotary_half(_rms(F.linear(x, w[p + "k_proj"]).view(s, -1, d), w[p + "k_norm"], cfg.rms_norm_eps)[None], cos, sin)[0]
        c["k"] = torch.cat([c["k"], k])
        c["v"] = torch.cat([c["v"], F.linear(x, w[p + "v_proj"]).view(s, -1, d)])
        safe = sel.clamp_min(0).long()
        gk, gv = c["k"][safe], c["v"][safe]                                              # [S, width, Hkv, d]
        qh = q.view(s, cfg.num_kv_heads, cfg.num_heads // cfg.num_kv_heads, d)
        sc = torch.einsum("qkgd,qskd->qkgs", qh, gk) * d ** -0.5
        sc = sc.masked_fill((sel < 0)[:, None, None, :], float("-inf"))
        o = torch.einsum("qkgs,qskd->qkgd", sc.softmax(-1), gv).reshape(s, -1)
        return F.linear(o * torch.sigmoid(gate), w[p + "o_proj"])

    def _mlp(self, i: int, x: torch.Tensor) -> torch.Tensor:
        cfg, w, p = self.cfg, self.w, f"layers.{i}.mlp."
        val, idx = C.topk_softmax_router(x, w[p + "gate"], cfg.experts_per_token, cfg.norm_topk)
        out = torch.zeros_like(x)
        for e in range(cfg.num_experts):
            if p + f"experts.{e}.gate_proj" not in w:                                     # another rank's expert
                continue
            hit = (idx == e)
            rows = hit.any(-1)
            if rows.any():
                y = _swiglu(x[rows], w[p + f"experts.{e}.gate_proj"], w[p + f"experts.{e}.up_proj"], w[p + f"experts.{e}.down_proj"])
                out[rows] += y * (val * hit)[rows].sum(-1, keepdim=True)
        shared = _swiglu(x, w[p + "shared.gate_proj"], w[p + "shared.up_proj"], w[p + "shared.down_proj"])
        return out + torch.sigmoid(F.linear(x, w[p + "shared_gate"])) * shared

    # ---- forward
    @torch.no_grad()
    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        ids = ids.reshape(-1).long().cpu()
        s, past = ids.numel(), self.length
        if past + s > self.max_context:
            raise RuntimeError("sequence exceeds max_context")
        history = torch.cat([self.history, ids[None]], 1)
        h, hc, eps = cfg.hidden_size, cfg.hc_count, cfg.rms_norm_eps
        streams = w["embed"][ids].repeat(1, hc)                                          # [S, hc * H]
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
        return F.linear(final.float(), w["lm_head"])

    def prefill_cached(self, prompt: torch.Tensor, cache) -> tuple[torch.Tensor, int]:
        """Prefill through a ``runtime.prefix_cache.PrefixCache``: resume from the longest cached prefix of ``prompt``,
        compute the rest in pieces that end on the cache's snapshot boundaries and store a snapshot at each.  Returns
        (logits of the last prompt position [vocab], tokens taken from the cache)."""
        toks = [int(t) for t in prompt.reshape(-1)]
        self.reset()
        hit = cache.lookup(toks)
        reused = 0
        if hit is not None:
            self.restore(hit.snapshot)
            reused = hit.tokens
        logits, pos = None, reused
        for b in cache.boundaries(reused, len(toks)) + [len(toks)]:
            logits = self.forward(prompt.reshape(-1)[pos:b])
            pos = b
            if b < len(toks) and not cache.contains(toks, b):
                snap = self.snapshot()
                nbytes = sum(t.numel() * t.element_size() for c in snap["cache"] for t in c.values()) + \
                    sum(t.numel() * t.element_size() for t in snap["ple_conv"].values())
                cache.insert(toks, b, [], snap, nbytes)
        return logits[-1], reused

    def generate(self, prompt: torch.Tensor, max_new_tokens: int, chunk: int = 64) -> list[int]:
        self.reset()
        logits = None
        for s0 in range(0, prompt.numel(), chunk):
            logits = self.forward(prompt[s0:s0 + chunk])
        out = []
        for _ in range(max_new_tokens):
            tok = int(logits[-1].argmax())
            out.append(tok)
            if len(out) == max_new_tokens:
                break
            logits = self.forward(torch.tensor([tok]))
        return out


# ---------------------------------------------------------------------------------------------- tensor parallel
def shard_weights(cfg: Qwen4ExpConfig, w: dict[str, torch.Tensor], rank: int, world: int) -> tuple[Qwen4ExpConfig, dict]:
    """The slice of a checkpoint one tensor-parallel rank holds, and the configuration it runs with.

    DeltaNet value heads, attention heads (queries with their gates, KV heads) and the shared expert's intermediate
    width are split; the output projections take the matching columns, so every sub-layer yields a partial sum.  Routed
    experts go round-robin (``id % world``), the lm_head is split by vocabulary rows, and the hyper-connection mixers,
    the router, the sparse-attention indexer and the n-gram injection are replicated.
    Reference behaviour: src/models/qwen4_exp/model.py:292 (TPShard), moe.py:475-501 (expert id % world)."""
    assert cfg.linear_v_heads % world == 0 and cfg.num_heads % world == 0 and cfg.num_kv_heads % world == 0
    assert cfg.shared_intermediate % world == 0 and cfg.vocab_size % world == 0
    split_k = cfg.linear_k_heads % world == 0 and cfg.linear_k_heads >= world
    kh = cfg.linear_k_heads // world if split_k else cfg.linear_k_heads
    vh, hq, hkv, d = cfg.linear_v_heads // world, cfg.num_heads // world, cfg.num_kv_heads // world, cfg.head_dim
    if not split_k:
        assert vh % kh == 0 or kh % vh == 0
    import dataclasses
    rcfg = dataclasses.replace(cfg, linear_k_heads=kh, linear_v_heads=vh, num_heads=hq, num_kv_heads=hkv,
                               shared_intermediate=cfg.shared_intermediate // world, layer_types=list(cfg.layer_types))
    KD, VD = cfg.linear_k_heads * 128, cfg.linear_v_heads * 128
    kr = torch.arange(rank * kh * 128, (rank + 1) * kh * 128) if split_k else torch.arange(KD)
    if not split_k and cfg.linear_k_heads > 1:               # value head j reads key head j // (Hv / Hk): keep those
        per = cfg.linear_v_heads // cfg.linear_k_heads
        heads = sorted({(rank * vh + j) // per for j in range(vh)})
        kr = torch.cat([torch.arange(hd * 128, (hd + 1) * 128) for hd in heads])
        rcfg = dataclasses.replace(rcfg, linear_k_heads=len(heads))
    vr = torch.arange(rank * vh * 128, (rank + 1) * vh * 128)
    qkv_rows = torch.cat([kr, KD + kr, 2 * KD + vr])
    hv_rows = torch.arange(rank * vh, (rank + 1) * vh)
    out = {}
    for k, t in w.items():
        leaf = k.rsplit(".", 1)[-1]
        if ".linear_attn." in k:
            if leaf in ("in_proj_qkv", "conv1d"):
                t = t[qkv_rows]
            elif leaf == "in_proj_z":
                t = t[vr]
            elif leaf in ("in_proj_a", "in_proj_b", "A_log", "dt_bias"):
                t = t[hv_rows]
            elif leaf == "out_proj":
                t = t[:, vr]
        elif ".self_attn." in k:
            if leaf == "q_proj":
                t = t[rank * hq * 2 * d:(rank + 1) * hq * 2 * d]
            elif leaf in ("k_proj", "v_proj"):
                t = t[rank * hkv * d:(rank + 1) * hkv * d]
            elif leaf == "o_proj":
                t = t[:, rank * hq * d:(rank + 1) * hq * d]
        elif ".mlp.experts." in k:
            if int(k.split(".experts.")[1].split(".")[0]) % world != rank:
                continue
        elif ".mlp.shared." in k:
            n = cfg.shared_intermediate // world
            t = t[:, rank * n:(rank + 1) * n] if leaf == "down_proj" else t[rank * n:(rank + 1) * n]
        elif k == "lm_head":
            n = cfg.vocab_size // world
            t = t[rank * n:(rank + 1) * n]
        out[k] = t.contiguous()
    return rcfg, out


class Qwen4ExpTP:
    """``world`` ranks of one model stepped in lock-step in this process: every sub-layer's partial outputs are summed
    (the all-reduce), logits are concatenated (the all-gather).  The replicated parts run once, on rank 0's copy."""

    def __init__(self, cfg: Qwen4ExpConfig, weights: dict, world: int, max_context: int = 512):
        self.cfg, self.world = cfg, world
        self.ranks = [Qwen4ExpRef(*shard_weights(cfg, weights, r, world), max_context) for r in range(world)]

    def reset(self) -> None:
        for r in self.ranks:
            r.reset()

    @torch.no_grad()
    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        cfg, r0 = self.cfg, self.ranks[0]
        w = r0.w
        ids = ids.reshape(-1).long()
        s, past = ids.numel(), r0.length
        history = torch.cat([r0.history, ids[None]], 1)
        h, hc, eps = cfg.hidden_size, cfg.hc_count, cfg.rms_norm_eps
        streams = w["embed"][ids].repeat(1, hc)
        for i, lt in enumerate(cfg.layer_types):
            p = f"layers.{i}."
            if i in cfg.ple_layers:
                streams = streams + r0._ple(i, streams, history)
            mixed, inject = C.gated_residual(streams, w[p + "attn_hc.hc_norm"], w[p + "attn_hc.down"], w[p + "attn_hc.up"],
                                             w[p + "attn_hc.inject"], hc, h, eps)
            attn = sum(r._deltanet(i, mixed.float()) if lt == "linear" else r._qsa(i, mixed.float(), past) for r in self.ranks)
            streams = C.inject_into_streams(attn, streams, inject.float())
            mixed, inject = C.gated_residual(streams, w[p + "mlp_hc.hc_norm"], w[p + "mlp_hc.down"], w[p + "mlp_hc.up"],
                                             w[p + "mlp_hc.inject"], hc, h, eps)
            streams = C.inject_into_streams(sum(r._mlp(i, mixed.float()) for r in self.ranks), streams, inject.float())
        for r in self.ranks:
            r.length, r.history = past + s, history[:, -(cfg.ngram_size - 1):].clone()
        final = C.gated_residual(streams, w["final.hc_norm"], w["final.down"], w["final.up"], None, hc, h, eps).float()
        return torch.cat([F.linear(final, r.w["lm_head"]) for r in self.ranks], -1)
