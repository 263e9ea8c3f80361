"""DSpark block drafter for the Qwen hybrid target, fp32 on the host: from the last committed token it proposes
``block_size`` tokens in one pass of a small dense transformer, with a confidence per token.

What it computes (behaviour of the reference's device runtime, cpp_engine/engine/qwen_dspark.cpp:603-836, and its
kernels, cpp_engine/backends/cuda/kernels/qwen_dspark_ops.cu:63-246):

* ``append_target_taps``: the target's hidden states after a few chosen layers, concatenated per position
  ``[rows, n_taps * hidden]``, are projected to ``hidden`` (``fc``), normalised (``hidden_norm``) and pushed through
  every draft layer's ``k_proj`` / ``v_proj``; keys get the per-head norm and the rotary embedding of their position.
  That is the drafter's whole memory of the committed context: it keeps no hidden states of its own.
* ``propose(anchor)``: the block is the anchor token followed by ``block_size - 1`` mask tokens, embedded with the
  target's embedding table, at positions ``committed ..``.  Every layer attends over the committed context keys plus the
  block's own keys, with no causal mask inside the block; residual, SwiGLU MLP, final norm, the target's vocabulary
  head.  Row ``i`` then receives a low-rank bigram bias from the token chosen for row ``i - 1`` (the anchor for row 0):
  ``logits[i] += markov_w2 @ markov_w1[prev]``, arg-max, and so on down the block.  The confidence of row ``i`` is
  ``sigmoid(w . [normalised hidden_i, markov_w1[prev_i]] + b)``.
* Rotary embedding is full-width YaRN (``yarn_inv_freqs``; cos and sin are both scaled by the attention factor), the
  norms are plain ``x * rsqrt(mean x^2 + eps) * gamma``.

``QwenDSparkDrafter`` puts the drafter behind the ``propose(context, k)`` protocol of the host speculative loop
(``components/speculative.py``) with the cache-less host target (``reference_cpu/qwen_hybrid_ref.py``): the block is
verified in one target pass, the longest agreeing prefix is kept together with the target's next token, and the taps
of the kept rows are appended (reference: cpp_engine/engine/qwen_engine.cpp:3904-3995).  The output equals plain
greedy decoding.

Checkpoint layout read by ``load_dspark`` (cpp_engine/engine/qwen_dspark.cpp:199-262, 360-410): ``config.json`` with
``block_size``, ``markov_rank``, ``dflash_config.{mask_token_id,target_layer_ids}``, ``rope_parameters``; tensors
``fc.weight``, ``hidden_norm.weight``, ``norm.weight``, ``markov_head.markov_w{1,2}.weight``,
``confidence_head.proj.{weight,bias}`` and ``layers.N.*``.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path

import torch
import torch.nn.functional as F


@dataclass
class QwenDSparkConfig:
    hidden_size: int
    intermediate_size: int
    vocab_size: int
    num_hidden_layers: int = 5
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    block_size: int = 7
    mask_token_id: int = 0
    markov_rank: int = 256
    target_layer_ids: list[int] = field(default_factory=list)
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e7
    rope_factor: float = 32.0
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    original_max_position_embeddings: int = 8192
    attention_factor: float = 0.0            # 0: derive 0.1 * ln(factor) + 1

    def __post_init__(self):
        if self.attention_factor <= 0.0:
            self.attention_factor = 0.1 * math.log(self.rope_factor) + 1.0
        assert self.num_attention_heads % self.num_key_value_heads == 0 and self.head_dim % 2 == 0
        assert self.block_size >= 1 and self.markov_rank >= 1 and self.target_layer_ids

    @staticmethod
    def from_json(path: str | Path) -> "QwenDSparkConfig":
        raw = json.loads(Path(path).read_text())
        df, rope = raw["dflash_config"], raw["rope_parameters"]
        for key, want in (("hidden_act", "silu"), ("markov_head_type", "vanilla")):
            if raw.get(key, want) != want:
                raise ValueError(f"unsupported DSpark drafter: {key}={raw[key]!r}")
        if df.get("attention_mode", "gqa") != "gqa" or df.get("projector_type", "dspark") != "dspark":
            raise ValueError("unsupported DSpark drafter: attention_mode / projector_type")
        if raw.get("attention_bias", False):
            raise ValueError("unsupported DSpark drafter: attention_bias")
        if any(t != "full_attention" for t in raw.get("layer_types", [])):
            raise ValueError("unsupported DSpark drafter: every layer must be full attention")
        return QwenDSparkConfig(
            hidden_size=raw["hidden_size"], intermediate_size=raw["intermediate_size"], vocab_size=raw["vocab_size"],
            num_hidden_layers=raw["num_hidden_layers"], num_attention_heads=raw["num_attention_heads"],
            num_key_value_heads=raw["num_key_value_heads"], head_dim=raw["head_dim"], block_size=raw["block_size"],
            mask_token_id=df["mask_token_id"], markov_rank=raw["markov_rank"], target_layer_ids=list(df["target_layer_ids"]),
            rms_norm_eps=raw.get("rms_norm_eps", 1e-6), rope_theta=rope["rope_theta"], rope_factor=rope["factor"],
            beta_fast=rope["beta_fast"], beta_slow=rope["beta_slow"],
            original_max_position_embeddings=rope["original_max_position_embeddings"],
            attention_factor=float(rope.get("attention_factor", 0.0)))

    def to_json(self) -> dict:
        return {"architectures": ["DSparkDraftModel"], "hidden_size": self.hidden_size,
                "intermediate_size": self.intermediate_size, "vocab_size": self.vocab_size,
                "num_hidden_layers": self.num_hidden_layers, "num_attention_heads": self.num_attention_heads,
                "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim, "block_size": self.block_size,
                "markov_rank": self.markov_rank, "rms_norm_eps": self.rms_norm_eps, "hidden_act": "silu",
                "markov_head_type": "vanilla", "attention_bias": False, "enable_confidence_head": True,
                "confidence_head_with_markov": True, "num_target_layers": len(self.target_layer_ids),
                "layer_types": ["full_attention"] * self.num_hidden_layers,
                "dflash_config": {"mask_token_id": self.mask_token_id, "target_layer_ids": list(self.target_layer_ids),
                                  "attention_mode": "gqa", "projector_type": "dspark"},
                "rope_parameters": {"rope_type": "yarn", "rope_theta": self.rope_theta, "factor": self.rope_factor,
                                    "beta_fast": self.beta_fast, "beta_slow": self.beta_slow,
                                    "original_max_position_embeddings": self.original_max_position_embeddings,
                                    "attention_factor": self.attention_factor}}


def yarn_inv_freqs(cfg: QwenDSparkConfig) -> torch.Tensor:
    """Per-pair inverse frequencies [head_dim / 2]: pairs that turn fast keep the original frequency, slow pairs are
    divided by ``rope_factor``, with a linear ramp between the two correction dimensions."""
    dim = cfg.head_dim

    def correction_dim(rotations: float) -> float:
        return dim * math.log(cfg.original_max_position_embeddings / (rotations * 2.0 * math.pi)) / (2.0 * math.log(cfg.rope_theta))

    low = max(0.0, math.floor(correction_dim(cfg.beta_fast)))
    high = min(float(dim - 1), math.ceil(correction_dim(cfg.beta_slow)))
    den = 0.001 if low == high else high - low
    pair = torch.arange(dim // 2, dtype=torch.float64)
    extrap = 1.0 / (cfg.rope_theta ** (2.0 * pair / dim))
    ramp = ((pair - low) / den).clamp(0.0, 1.0)              # 0: keep, 1: interpolate
    return (extrap / cfg.rope_factor * ramp + extrap * (1.0 - ramp)).float()


def _norm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * gamma


def _rope(x: torch.Tensor, start: int, inv: torch.Tensor, factor: float) -> torch.Tensor:
    """x [rows, heads, head_dim]; pair ``p`` is (x[p], x[half + p])."""
    rows, half = x.shape[0], x.shape[-1] // 2
    ang = (torch.arange(rows, dtype=torch.float32) + start)[:, None] * inv[None, :]
    cos, sin = (ang.cos() * factor)[:, None, :], (ang.sin() * factor)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)


def expected_tensors(cfg: QwenDSparkConfig) -> dict[str, tuple[int, ...]]:
    """Name -> shape of every tensor of a drafter checkpoint (7 global + 11 per layer)."""
    h, inter, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    qd, kvd = cfg.num_attention_heads * d, cfg.num_key_value_heads * d
    t = {"fc.weight": (h, h * len(cfg.target_layer_ids)), "hidden_norm.weight": (h,), "norm.weight": (h,),
         "markov_head.markov_w1.weight": (cfg.vocab_size, cfg.markov_rank),
         "markov_head.markov_w2.weight": (cfg.vocab_size, cfg.markov_rank),
         "confidence_head.proj.weight": (1, h + cfg.markov_rank), "confidence_head.proj.bias": (1,)}
    for i in range(cfg.num_hidden_layers):
        p = f"layers.{i}."
        t.update({p + "input_layernorm.weight": (h,), p + "post_attention_layernorm.weight": (h,),
                  p + "self_attn.q_proj.weight": (qd, h), p + "self_attn.k_proj.weight": (kvd, h),
                  p + "self_attn.v_proj.weight": (kvd, h), p + "self_attn.o_proj.weight": (h, qd),
                  p + "self_attn.q_norm.weight": (d,), p + "self_attn.k_norm.weight": (d,),
                  p + "mlp.gate_proj.weight": (inter, h), p + "mlp.up_proj.weight": (inter, h),
                  p + "mlp.down_proj.weight": (h, inter)})
    return t


def synth_dspark_weights(cfg: QwenDSparkConfig, seed: int = 0, std: float = 0.05) -> dict[str, torch.Tensor]:
    """Seeded random drafter in checkpoint dtype (bf16): norms near 1, matrices N(0, std), the bigram and confidence
    tables wider so that they change the arg-max in tests."""
    g = torch.Generator().manual_seed(seed + 991)
    w = {}
    for name, shape in expected_tensors(cfg).items():
        if name.endswith(("norm.weight", "layernorm.weight")):
            w[name] = (1.0 + torch.randn(*shape, generator=g) * 0.05).to(torch.bfloat16)
        else:
            sd = 0.3 if name.startswith(("markov_head", "confidence_head")) else std
            w[name] = (torch.randn(*shape, generator=g) * sd).to(torch.bfloat16)
    return w


def load_dspark(directory: str | Path) -> tuple[QwenDSparkConfig, dict[str, torch.Tensor]]:
    """Read a drafter checkpoint directory; checks names and shapes against the configuration."""
    from ..formats import safetensors_io
    directory = Path(directory)
    cfg = QwenDSparkConfig.from_json(directory / "config.json")
    w = {k: v for k, v in safetensors_io.read_checkpoint(str(directory))}
    want = expected_tensors(cfg)
    missing = sorted(set(want) - set(w))
    extra = sorted(set(w) - set(want))
    if missing or extra:
        raise ValueError(f"DSpark checkpoint does not hold exactly the expected {len(want)} tensors: "
                         f"missing {missing[:4]}, unexpected {extra[:4]}")
    for k, shape in want.items():
        if tuple(w[k].shape) != shape:
            raise ValueError(f"DSpark tensor {k}: shape {tuple(w[k].shape)}, expected {shape}")
    return cfg, w


@dataclass
class DSparkProposal:
    tokens: list[int]
    confidences: list[float]
    top_logits: list[float]


class QwenDSparkRef:
    """``embedding`` [vocab, hidden] and ``head`` [vocab, hidden] are the target's tables (shared, not copied)."""

    def __init__(self, cfg: QwenDSparkConfig, weights: dict[str, torch.Tensor], embedding: torch.Tensor,
                 head: torch.Tensor, max_context: int = 4096):
        self.cfg, self.max_context = cfg, max_context
        self.w = {k: v.float() for k, v in weights.items()}
        self.embedding, self.head = embedding.float(), head.float()
        if self.embedding.shape != (cfg.vocab_size, cfg.hidden_size) or self.head.shape != self.embedding.shape:
            raise ValueError("DSpark drafter does not match the target's embedding / head")
        self.inv = yarn_inv_freqs(cfg)
        kvd = cfg.num_key_value_heads * cfg.head_dim
        self.ctx_k = [torch.zeros(max_context, kvd) for _ in range(cfg.num_hidden_layers)]
        self.ctx_v = [torch.zeros(max_context, kvd) for _ in range(cfg.num_hidden_layers)]
        self.committed = 0

    # -- context
    def reset(self) -> None:
        self.committed = 0

    def crop_context(self, position: int) -> None:
        if not 0 <= position <= self.committed:
            raise ValueError("invalid DSpark context crop")
        self.committed = position

    @torch.no_grad()
    def append_target_taps(self, taps: torch.Tensor, position_offset: int) -> None:
        cfg, w = self.cfg, self.w
        rows = taps.shape[0]
        if rows <= 0 or position_offset != self.committed or position_offset + rows > self.max_context \
                or taps.shape[1] != cfg.hidden_size * len(cfg.target_layer_ids):
            raise ValueError("invalid DSpark target tap append")
        ctx = _norm(taps.float() @ w["fc.weight"].t(), w["hidden_norm.weight"], cfg.rms_norm_eps)
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}.self_attn."
            k = (ctx @ w[p + "k_proj.weight"].t()).view(rows, cfg.num_key_value_heads, cfg.head_dim)
            k = _rope(_norm(k, w[p + "k_norm.weight"], cfg.rms_norm_eps), position_offset, self.inv, cfg.attention_factor)
            self.ctx_k[i][position_offset:position_offset + rows] = k.reshape(rows, -1)
            self.ctx_v[i][position_offset:position_offset + rows] = ctx @ w[p + "v_proj.weight"].t()
        self.committed += rows

    # -- one block
    @torch.no_grad()
    def block_hidden(self, anchor: int) -> torch.Tensor:
        """Final-normed hidden rows [block_size, hidden] of the block that starts with ``anchor``."""
        cfg, w, eps = self.cfg, self.w, self.cfg.rms_norm_eps
        if not 0 <= anchor < cfg.vocab_size or self.committed >= self.max_context:
            raise ValueError("invalid DSpark proposal anchor")
        b, hq, hkv, d, n = cfg.block_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, self.committed
        ids = torch.full((b,), cfg.mask_token_id, dtype=torch.long)
        ids[0] = anchor
        h = self.embedding[ids]
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}."
            x = _norm(h, w[p + "input_layernorm.weight"], eps)
            q = (x @ w[p + "self_attn.q_proj.weight"].t()).view(b, hq, d)
            k = (x @ w[p + "self_attn.k_proj.weight"].t()).view(b, hkv, d)
            v = (x @ w[p + "self_attn.v_proj.weight"].t()).view(b, hkv, d)
            q = _rope(_norm(q, w[p + "self_attn.q_norm.weight"], eps), n, self.inv, cfg.attention_factor)
            k = _rope(_norm(k, w[p + "self_attn.k_norm.weight"], eps), n, self.inv, cfg.attention_factor)
            keys = torch.cat([self.ctx_k[i][:n].view(n, hkv, d), k], 0).repeat_interleave(hq // hkv, 1)
            vals = torch.cat([self.ctx_v[i][:n].view(n, hkv, d), v], 0).repeat_interleave(hq // hkv, 1)
            s = torch.einsum("qhd,khd->hqk", q, keys) / math.sqrt(d)        # no mask: the block sees all of itself
            o = torch.einsum("hqk,khd->qhd", s.softmax(-1), vals).reshape(b, hq * d)
            h = h + o @ w[p + "self_attn.o_proj.weight"].t()
            x = _norm(h, w[p + "post_attention_layernorm.weight"], eps)
            act = F.silu(x @ w[p + "mlp.gate_proj.weight"].t()) * (x @ w[p + "mlp.up_proj.weight"].t())
            h = h + act @ w[p + "mlp.down_proj.weight"].t()
        return _norm(h, w["norm.weight"], eps)

    @torch.no_grad()
    def propose(self, anchor: int) -> DSparkProposal:
        cfg, w = self.cfg, self.w
        x = self.block_hidden(anchor)
        logits = x @ self.head.t()
        tokens, tops, prev, emb = [], [], anchor, []
        for row in range(cfg.block_size):
            e = w["markov_head.markov_w1.weight"][prev]
            emb.append(e)
            logits[row] += w["markov_head.markov_w2.weight"] @ e
            prev = int(logits[row].argmax())
            tokens.append(prev)
            tops.append(float(logits[row, prev]))
        feat = torch.cat([x, torch.stack(emb)], -1)
        conf = torch.sigmoid(feat @ w["confidence_head.proj.weight"][0] + w["confidence_head.proj.bias"][0])
        return DSparkProposal(tokens, [float(c) for c in conf], tops)


class QwenDSparkDrafter:
    """The drafter behind the ``propose(context, k)`` protocol of ``components/speculative.py``.  ``target`` is the
    ``WholeSequenceTarget`` of a ``QwenHybridRef``; its ``capture_layers`` are set to the drafter's tap layers, and
    before every proposal the taps of the context rows that the drafter has not seen yet are appended.  Rows of a
    rejected block never reach the drafter: only the committed context is appended, so nothing has to be cropped."""

    def __init__(self, target, drafter: QwenDSparkRef):
        self.t, self.d = target, drafter
        target.oracle.capture_layers = tuple(drafter.cfg.target_layer_ids)

    def propose(self, context: list[int], k: int) -> tuple[list[int], list[float]]:
        taps = getattr(self.t, "taps", None)
        n = len(context) - 1                                    # rows the target has run: everything before the anchor
        if k <= 0 or taps is None or taps.shape[0] < n or n + self.d.cfg.block_size > self.d.max_context:
            return [], []
        if self.d.committed > n:                                # a new sequence
            self.d.reset()
        if self.d.committed < n:
            self.d.append_target_taps(taps[self.d.committed:n], self.d.committed)
        prop = self.d.propose(context[-1])
        return prop.tokens[:k], prop.confidences[:k]
