"""The full DeepSeek-V4-style decoder assembled from ``v4_components`` as an fp32 CPU runtime with caches: Sinkhorn
hyper-connection streams around every sub-layer, multi-query latent attention over a sliding-window ring plus learned
compressed KV entries (ratio-4 layers pick their compressed entries with the Hadamard-rotated indexer, other ratios
take every complete entry), attention sink, inverse rotary on the output, grouped low-rank output projection, hash-routed
and score-routed experts with a clamped SwiGLU and a shared expert, the hyper-connection head and the depth-1 MTP
block.  It is the executable statement of that block for tiny configurations; the 8-bit / 4-bit activation fake-quant of
the trained model is left out (fp32 throughout).  The served DSV4 shape on the GPU is ``models/mla_moe_gpu.py``.

Reference behaviour (src/models/deepseek_v4/runtime.py): Indexer :1112-1288, Attention :1291-1660, Gate :1662-1731,
Expert clamp :2267-2269, Block :4277-4497, ParallelHead.hc_head :4597-4607, MTPBlock :4610-4642, Transformer :4645-4922.
A prompt is processed in one pass from position 0 and continued token by token, as there.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import v4_components as V


@dataclass
class V4Config:
    vocab_size: int = 200
    dim: int = 64
    n_layers: int = 3
    n_heads: int = 4
    head_dim: int = 32
    rope_head_dim: int = 16
    q_lora_rank: int = 32
    o_groups: int = 2
    o_lora_rank: int = 16
    window: int = 8
    compress_ratios: tuple[int, ...] = (0, 4, 8)        # per layer: 0 = window only, 4 = indexer-selected, else all complete
    index_n_heads: int = 4
    index_head_dim: int = 128                           # the Hadamard rotation is 128 wide
    index_topk: int = 3
    hc_mult: int = 4
    hc_iters: int = 20
    hc_eps: float = 1e-6
    n_experts: int = 4
    n_activated: int = 2
    n_shared: int = 1
    moe_inter: int = 32
    n_hash_layers: int = 1
    score_func: str = "sqrtsoftplus"
    route_scale: float = 1.5
    swiglu_limit: float = 7.0
    rope_theta: float = 10000.0
    compress_rope_theta: float = 40000.0
    rope_factor: float = 4.0
    original_seq_len: int = 64
    norm_eps: float = 1e-6
    max_seq_len: int = 256
    mtp: bool = True

    def __post_init__(self):
        assert len(self.compress_ratios) == self.n_layers and self.n_heads % self.o_groups == 0
        assert self.rope_head_dim <= self.head_dim and self.index_head_dim == 128


def _layer_weights(cfg: V4Config, r, one, p: str, ratio: int, hashed: bool) -> dict[str, torch.Tensor]:
    d, hc = cfg.dim, cfg.hc_mult
    w = {}
    for blk in ("attn", "ffn"):
        w[p + f"hc_{blk}_fn"] = r((2 + hc) * hc, hc * d)
        w[p + f"hc_{blk}_scale"], w[p + f"hc_{blk}_base"] = one(3), r((2 + hc) * hc, sd=0.3)
        w[p + f"{blk}_norm"] = one(d)
    a = p + "attn."
    w[a + "wq_a"], w[a + "q_norm"] = r(cfg.q_lora_rank, d), one(cfg.q_lora_rank)
    w[a + "wq_b"] = r(cfg.n_heads * cfg.head_dim, cfg.q_lora_rank, sd=0.15)
    w[a + "wkv"], w[a + "kv_norm"] = r(cfg.head_dim, d, sd=0.15), one(cfg.head_dim)
    w[a + "attn_sink"] = r(cfg.n_heads, sd=0.5)
    w[a + "wo_a"] = r(cfg.o_groups * cfg.o_lora_rank, cfg.n_heads // cfg.o_groups * cfg.head_dim, sd=0.1)
    w[a + "wo_b"] = r(d, cfg.o_groups * cfg.o_lora_rank, sd=0.1)
    if ratio:
        coff = 2 if ratio == 4 else 1
        c = a + "compressor."
        w[c + "wkv"], w[c + "wgate"] = r(coff * cfg.head_dim, d, sd=0.15), r(coff * cfg.head_dim, d, sd=0.15)
        w[c + "ape"], w[c + "norm"] = r(ratio, coff * cfg.head_dim, sd=0.3), one(cfg.head_dim)
    if ratio == 4:
        i, di = a + "indexer.", cfg.index_head_dim
        w[i + "wq_b"] = r(cfg.index_n_heads * di, cfg.q_lora_rank, sd=0.15)
        w[i + "weights_proj"] = r(cfg.index_n_heads, d, sd=0.3)
        c = i + "compressor."
        w[c + "wkv"], w[c + "wgate"] = r(2 * di, d, sd=0.15), r(2 * di, d, sd=0.15)
        w[c + "ape"], w[c + "norm"] = r(ratio, 2 * di, sd=0.3), one(di)
    f = p + "ffn."
    w[f + "gate"] = r(cfg.n_experts, d, sd=0.3)
    if hashed:
        g = torch.Generator().manual_seed(len(p))
        w[f + "tid2eid"] = torch.stack([torch.randperm(cfg.n_experts, generator=g)[:cfg.n_activated] for _ in range(cfg.vocab_size)])
    else:
        w[f + "gate_bias"] = r(cfg.n_experts, sd=0.3)
    for e in [str(k) for k in range(cfg.n_experts)] + ["shared"]:
        inter = cfg.moe_inter * (cfg.n_shared if e == "shared" else 1)
        w[f + f"experts.{e}.w1"], w[f + f"experts.{e}.w3"] = r(inter, d, sd=0.15), r(inter, d, sd=0.15)
        w[f + f"experts.{e}.w2"] = r(d, inter, sd=0.15)
    return w


def synth_weights(cfg: V4Config, seed: int = 0) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, sd=0.05: torch.randn(*s, generator=g) * sd
    one = lambda *s: 1.0 + r(*s, sd=0.05)
    d, hc = cfg.dim, cfg.hc_mult
    w = {"embed": r(cfg.vocab_size, d, sd=0.5), "head": r(cfg.vocab_size, d, sd=0.1), "norm": one(d),
         "hc_head_fn": r(hc, hc * d), "hc_head_scale": one(1), "hc_head_base": r(hc, sd=0.3)}
    for i, ratio in enumerate(cfg.compress_ratios):
        w.update(_layer_weights(cfg, r, one, f"layers.{i}.", ratio, i < cfg.n_hash_layers))
    if cfg.mtp:
        p = "mtp."
        w.update(_layer_weights(cfg, r, one, p, 0, False))
        w[p + "e_proj"], w[p + "h_proj"] = r(d, d, sd=0.1), r(d, d, sd=0.1)
        w[p + "enorm"], w[p + "hnorm"], w[p + "norm"] = one(d), one(d), one(d)
        w[p + "hc_head_fn"], w[p + "hc_head_scale"], w[p + "hc_head_base"] = r(hc, hc * d), one(1), r(hc, sd=0.3)
    return w


def _rms(x: torch.Tensor, g: torch.Tensor | None, eps: float) -> torch.Tensor:
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return y if g is None else y * g


def sparse_attention_ref(q: torch.Tensor, kv: torch.Tensor, sink: torch.Tensor, idx: torch.Tensor, scale: float) -> torch.Tensor:
    """q [S, H, D], kv [N, D] (keys and values are the same rows), sink [H] a per-head logit that only enlarges the
    soft-max denominator, idx [S, K] rows of ``kv`` per query (-1 = none) -> [S, H, D]."""
    g = kv[idx.clamp_min(0).long()]                                                     # [S, K, D]
    sc = torch.einsum("shd,skd->shk", q, g) * scale
    sc = sc.masked_fill((idx < 0)[:, None, :], float("-inf"))
    m = torch.maximum(sc.amax(-1), sink[None, :])                                       # [S, H]
    p = torch.exp(sc - m[..., None])
    den = p.sum(-1) + torch.exp(sink[None, :] - m)
    return torch.einsum("shk,skd->shd", p / den[..., None], g)


class _Layer:
    """Caches of one block: window ring + compressed rows, the KV compressor and the indexer's own compressor / keys."""

    def __init__(self, cfg: V4Config, w: dict, p: str, ratio: int, hashed: bool):
        self.cfg, self.w, self.p, self.ratio, self.hashed = cfg, w, p, ratio, hashed
        theta, factor, orig = (cfg.compress_rope_theta, cfg.rope_factor, cfg.original_seq_len) if ratio else (cfg.rope_theta, 1.0, 0)
        self.table = V.rotary_table(cfg.rope_head_dim, cfg.max_seq_len, theta, factor, orig)
        # hooks of the long-context runtime (models/v4_flashmemory.py), ratio-4 layers only
        self.global_pick: torch.Tensor | None = None     # compressed entries chosen for this decode step by a shared retriever
        self.store = None                                # home of the compressed rows outside this layer (host pool + working set)
        self.reset()

    def reset(self) -> None:
        cfg, w, a, r = self.cfg, self.w, self.p + "attn.", self.ratio
        self.kv = torch.zeros(cfg.window + (cfg.max_seq_len // r if r and self.store is None else 0), cfg.head_dim)
        self.comp = self.icomp = None
        if r:
            c = a + "compressor."
            self.comp = V.Compressor(w[c + "wkv"], w[c + "wgate"], w[c + "ape"], w[c + "norm"], r, cfg.head_dim, cfg.rope_head_dim,
                                     self.table, cfg.norm_eps)
        if r == 4:
            c = a + "indexer.compressor."
            self.icomp = V.Compressor(w[c + "wkv"], w[c + "wgate"], w[c + "ape"], w[c + "norm"], r, cfg.index_head_dim,
                                      cfg.rope_head_dim, self.table, cfg.norm_eps)
            self.ikeys = torch.zeros(cfg.max_seq_len // r, cfg.index_head_dim)

    # ---- indexer: compressed entries of a ratio-4 layer chosen per query
    def _index(self, x: torch.Tensor, qr: torch.Tensor, start: int, offset: int) -> torch.Tensor:
        cfg, w, i, r = self.cfg, self.w, self.p + "attn.indexer.", self.ratio
        s, rd, end = x.shape[0], cfg.rope_head_dim, start + x.shape[0]
        q = (qr @ w[i + "wq_b"].t()).view(1, s, cfg.index_n_heads, cfg.index_head_dim)
        q = torch.cat([q[..., :-rd], V.apply_rotary(q[..., -rd:].contiguous(), self.table[start:end])], -1)
        q = V.hadamard128_ref(q)[0]
        new = self.icomp.forward(x[None], start)
        if new is not None:
            n0 = 0 if start == 0 else start // r
            self.ikeys[n0:n0 + new.shape[1]] = V.hadamard128_ref(new[0])
        heads_w = (x @ w[i + "weights_proj"].t()) * (cfg.index_head_dim ** -0.5 * cfg.index_n_heads ** -0.5)
        keys = self.ikeys[:end // r]
        score = (torch.relu(torch.einsum("shd,td->sht", q, keys)) * heads_w[..., None]).sum(1)      # [S, t]
        valid = ((start + torch.arange(s) + 1) // r)[:, None]
        score = score.masked_fill(torch.arange(keys.shape[0])[None, :] >= valid, float("-inf"))
        k = min(cfg.index_topk, end // r)
        # ties (all-zero relu rows) go to the earlier entry, so the choice does not depend on how many later ones exist
        pick = torch.sort(score, dim=-1, descending=True, stable=True).indices[:, :k]
        return torch.where(pick >= valid, torch.full_like(pick, -1), pick + offset)

    def attention(self, x: torch.Tensor, start: int) -> torch.Tensor:
        cfg, w, a, r, win = self.cfg, self.w, self.p + "attn.", self.ratio, self.cfg.window
        s, rd, end = x.shape[0], cfg.rope_head_dim, start + x.shape[0]
        assert start == 0 or s == 1
        tab = self.table[start:end]
        qr = _rms(x @ w[a + "wq_a"].t(), w[a + "q_norm"], cfg.norm_eps)
        q = _rms((qr @ w[a + "wq_b"].t()).view(1, s, cfg.n_heads, cfg.head_dim), None, cfg.norm_eps)
        q = torch.cat([q[..., :-rd], V.apply_rotary(q[..., -rd:].contiguous(), tab)], -1)[0]
        kv = _rms(x @ w[a + "wkv"].t(), w[a + "kv_norm"], cfg.norm_eps)[None]
        kv = torch.cat([kv[..., :-rd], V.apply_rotary(kv[..., -rd:].contiguous(), tab)], -1)[0]
        idx = V.window_indices(win, s, start)
        comp_idx = None
        if r:
            offset = s if start == 0 else win
            comp_idx = self._index(x, qr, start, offset) if r == 4 else V.compressed_indices(r, s, start, offset)
            if r == 4 and self.global_pick is not None and start > 0:
                g = self.global_pick.long().reshape(1, -1)
                if int(g.max()) >= end // r:
                    raise RuntimeError("the shared selection names a compressed entry this layer does not have yet")
                comp_idx = torch.where(g < 0, g, g + offset)
        if start == 0:
            if s <= win:
                self.kv[:s] = kv
            else:
                cut = s % win
                self.kv[cut:win], self.kv[:cut] = kv[-win:].split([win - cut, cut])
            rows = kv
            if r and (new := self.comp.forward(x[None], 0)) is not None:
                if self.store is None:
                    self.kv[win:win + new.shape[1]] = new[0]
                else:
                    for j in range(new.shape[1]):
                        self.store.append(j, new[0, j])
                rows = torch.cat([kv, new[0]])
        else:
            self.kv[start % win] = kv[0]
            new = self.comp.forward(x[None], start) if r else None
            if self.store is None:
                if new is not None:
                    self.kv[win + start // r] = new[0, 0]
                rows = self.kv
            else:
                if new is not None:
                    self.store.append(start // r, new[0, 0])
                entries = torch.where(comp_idx < 0, comp_idx, comp_idx - offset)[0]
                rows = torch.cat([self.kv[:win], self.store.gather(entries)])
                comp_idx = torch.where(entries < 0, entries, win + torch.arange(entries.numel()))[None, :]
        if comp_idx is not None:
            idx = torch.cat([idx, comp_idx], -1)
        o = sparse_attention_ref(q, rows, w[a + "attn_sink"], idx, cfg.head_dim ** -0.5)
        o = torch.cat([o[..., :-rd], V.apply_rotary(o[None, ..., -rd:].contiguous(), tab, inverse=True)[0]], -1)
        o = torch.einsum("sgd,grd->sgr", o.reshape(s, cfg.o_groups, -1), w[a + "wo_a"].view(cfg.o_groups, cfg.o_lora_rank, -1))
        return o.flatten(1) @ w[a + "wo_b"].t()

    def ffn(self, x: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        cfg, w, f = self.cfg, self.w, self.p + "ffn."
        wts, idx = V.gate_route(x, w[f + "gate"], None if self.hashed else w[f + "gate_bias"], cfg.n_activated, cfg.score_func,
                                cfg.route_scale, w[f + "tid2eid"] if self.hashed else None, ids if self.hashed else None)
        lim = cfg.swiglu_limit

        def expert(e, t, clamp):
            gate, up = t @ w[f + f"experts.{e}.w1"].t(), t @ w[f + f"experts.{e}.w3"].t()
            if clamp and lim > 0:
                gate, up = gate.clamp(max=lim), up.clamp(-lim, lim)
            return (F.silu(gate) * up) @ w[f + f"experts.{e}.w2"].t()

        y = expert("shared", x, False)
        for e in range(cfg.n_experts):
            hit = idx == e
            rows = hit.any(-1)
            if rows.any():
                y[rows] += expert(e, x[rows], True) * (wts * hit)[rows].sum(-1, keepdim=True)
        return y

    def forward(self, streams: torch.Tensor, start: int, ids: torch.Tensor) -> torch.Tensor:
        """streams [S, hc, D]."""
        cfg, w, p = self.cfg, self.w, self.p
        for blk, fn in (("attn", lambda t: self.attention(t, start)), ("ffn", lambda t: self.ffn(t, ids))):
            y, post, comb = V.hc_pre(streams[None], w[p + f"hc_{blk}_fn"], w[p + f"hc_{blk}_scale"], w[p + f"hc_{blk}_base"],
                                     cfg.norm_eps, cfg.hc_iters, cfg.hc_eps)
            y = fn(_rms(y[0], w[p + f"{blk}_norm"], cfg.norm_eps))
            streams = V.hc_post(y[None], streams[None], post, comb)[0]
        return streams


class V4BlockRef:
    """One sequence, fp32, CPU.  ``forward(ids)`` takes the whole prompt at position 0 or one token after it and returns
    logits [S, vocab]; ``draft(ids)`` runs the MTP block on the hidden streams of the last ``forward`` and the tokens that
    follow each of its positions, returning the logits of the position after those."""

    def __init__(self, cfg: V4Config, weights: dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, {k: (v.float() if v.is_floating_point() else v) for k, v in weights.items()}
        self.layers = [_Layer(cfg, self.w, f"layers.{i}.", r, i < cfg.n_hash_layers) for i, r in enumerate(cfg.compress_ratios)]
        self.mtp = _Layer(cfg, self.w, "mtp.", 0, False) if cfg.mtp else None
        self.reset()

    def reset(self) -> None:
        self.length, self.hidden, self.layer_hidden = 0, None, []
        for l in self.layers + ([self.mtp] if self.mtp else []):
            l.reset()

    _STATE = ("kv", "ikeys")

    def snapshot(self) -> dict:
        """Everything positional a prefix cache must keep: per layer the window ring + compressed rows, the running
        state of the KV compressor and of the indexer's compressor, and the indexer keys."""
        import copy
        layers = []
        for l in self.layers + ([self.mtp] if self.mtp else []):
            st = {k: getattr(l, k).clone() for k in self._STATE if hasattr(l, k)}
            for name in ("comp", "icomp"):
                c = getattr(l, name)
                if c is not None:
                    st[name] = (c.kv_state.clone(), c.score_state.clone())
            layers.append(st)
        return {"length": self.length, "layers": layers, "hidden": copy.deepcopy(self.hidden),
                "layer_hidden": [h.clone() for h in self.layer_hidden]}

    def restore(self, snap: dict) -> None:
        self.length = snap["length"]
        self.hidden = None if snap["hidden"] is None else snap["hidden"].clone()
        self.layer_hidden = [h.clone() for h in snap["layer_hidden"]]
        for l, st in zip(self.layers + ([self.mtp] if self.mtp else []), snap["layers"]):
            for k in self._STATE:
                if k in st:
                    setattr(l, k, st[k].clone())
            for name in ("comp", "icomp"):
                if name in st:
                    c = getattr(l, name)
                    c.kv_state, c.score_state = st[name][0].clone(), st[name][1].clone()

    def _head(self, streams: torch.Tensor, p: str) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        flat = streams.flatten(1)
        mixes = (flat @ w[p + "hc_head_fn"].t()) * torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + cfg.norm_eps)
        pre = torch.sigmoid(mixes * w[p + "hc_head_scale"] + w[p + "hc_head_base"]) + cfg.hc_eps
        y = (pre[..., None] * streams).sum(1)
        return _rms(y, w[p + "norm"], cfg.norm_eps) @ w["head"].t()

    @torch.no_grad()
    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        ids = ids.reshape(-1).long()
        s, start = ids.numel(), self.length
        if start + s > cfg.max_seq_len:
            raise RuntimeError("sequence exceeds max_seq_len")
        if start > 0 and s != 1:
            raise RuntimeError("a started sequence continues one token at a time")
        streams = self.w["embed"][ids][:, None, :].repeat(1, cfg.hc_mult, 1)              # [S, hc, D]
        self.layer_hidden = []                                                            # per layer [S, D]: mean over the streams
        for l in self.layers:
            streams = l.forward(streams, start, ids)
            self.layer_hidden.append(streams.mean(1))
        self.hidden, self.length = streams, start + s
        return self._head(streams, "")

    @torch.no_grad()
    def draft(self, next_ids: torch.Tensor) -> torch.Tensor:
        """next_ids [S]: the token after each position of the last ``forward`` call."""
        cfg, w, p = self.cfg, self.w, "mtp."
        assert self.mtp is not None and self.hidden is not None
        next_ids = next_ids.reshape(-1).long()
        s = self.hidden.shape[0]
        assert next_ids.numel() == s
        start = self.length - s
        e = _rms(w["embed"][next_ids], w[p + "enorm"], cfg.norm_eps) @ w[p + "e_proj"].t()
        h = _rms(self.hidden, w[p + "hnorm"], cfg.norm_eps) @ w[p + "h_proj"].t()
        streams = self.mtp.forward(e[:, None, :] + h, start, next_ids)
        return self._head(streams, p)

    def generate(self, prompt: torch.Tensor, max_new_tokens: int) -> list[int]:
        self.reset()
        logits, out = self.forward(prompt), []
        for _ in range(max_new_tokens):
            out.append(int(logits[-1].argmax()))
            if len(out) < max_new_tokens:
                logits = self.forward(torch.tensor([out[-1]]))
        return out

    def generate_speculative(self, prompt: torch.Tensor, max_new_tokens: int) -> tuple[list[int], int]:
        """Greedy decoding with the MTP block proposing one token ahead: returns the tokens (identical to ``generate``)
        and how many proposals matched.  The proposal is only scored here, not used to skip a step."""
        self.reset()
        logits, out, hits, proposal = self.forward(prompt), [], 0, None
        prev = prompt.reshape(-1).long()
        for _ in range(max_new_tokens):
            tok = int(logits[-1].argmax())
            hits += int(proposal is not None and proposal == tok)
            out.append(tok)
            if len(out) == max_new_tokens:
                break
            nxt = torch.cat([prev[1:], torch.tensor([tok])]) if self.hidden.shape[0] == prev.numel() else torch.tensor([tok])
            proposal = int(self.draft(nxt)[-1].argmax())
            prev = torch.tensor([tok])
            logits = self.forward(prev)
        return out, hits
