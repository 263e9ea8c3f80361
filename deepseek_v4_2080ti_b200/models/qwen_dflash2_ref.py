"""DFlash2 block-diffusion drafter for the Qwen hybrid target, fp32 on the host: one denoising pass over a block of
``block_size`` rows (the committed anchor followed by mask tokens) yields ``block_size - 1`` drafts, chosen from the
top-k candidates of every row by a low-rank pairwise selector.

What it computes (behaviour of the reference's device runtime, cpp_engine/engine/qwen_dflash2.cpp:770-1260, and its
kernels, cpp_engine/backends/cuda/kernels/qwen_dflash2_ops.cu:82-277 and 598-848):

* Context memory as in the DSpark drafter: target taps -> ``fc`` -> ``hidden_norm`` -> per layer ``k_proj`` (head norm,
  rotary embedding at the row's position) and ``v_proj``.  Plain rotary embedding over the whole head, no scaling.
* Each of the two branches of a layer is wrapped in a *dynamic grouped convolution* over the block's rows: from the
  normalised input, ``kernel_projection`` produces per row ``2 * K * groups`` tap offsets; the first half shapes the
  convolution in front of the branch (``prepare``), the second half the one behind it (``finish``).  A convolution is
  ``y[row, c] = sum_tap x[row - tap, c] * (base[tap, c] + dyn[row, tap * groups + c // group_size])`` with rows before
  the block reading zero.
* Attention over the committed context plus the block, without a causal mask inside the block, limited to keys with
  ``|query position - key position| < sliding_window``.
* The residual stream stays in fp32; the final norm of rows ``1 ..`` goes through the target's vocabulary head.  Every
  draft row keeps its ``selector_top_k`` best tokens (ties: the lower token id) and their logits as unary scores.  The
  selector scores a step from token ``a`` to candidate ``b`` at row ``i`` as
  ``unary[i, b] + sum_r predecessor[a, r] * (hidden_i @ P^T)[r] * successor[b, r]`` and picks either greedily down the
  block (each row conditioned on the previous pick, the anchor first) or the best whole path (Viterbi).
* ``refine_passes > 1`` feeds the drafts back in place of the mask tokens and runs the pass again until they stop
  changing.
* ``debug`` (a callable) receives every intermediate stage under the names the reference's debug view uses
  (``context.projected`` ... ``layer.N.attention.q_rope`` ... ``selector.path``, cpp_engine/engine/qwen_dflash2.cpp:
  667-724 and the ``dump_*`` calls), which is what ``cli/check_drafter_fixture.py`` compares with an exported fixture.

Checkpoint names (cpp_engine/engine/qwen_dflash2.cpp:450-482): ``fc.weight``, ``hidden_norm.weight``, ``norm.weight``,
``candidate_selector.{predecessor_codebook,successor_codebook,hidden_projection.weight}`` and per layer the eleven
transformer tensors plus ``{attention_conv,mlp_conv}.{base_kernel,kernel_projection.weight}``.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path

import torch
import torch.nn.functional as F

from ..components import draft_selector as sel
from .qwen_dspark_ref import _norm


@dataclass
class QwenDFlash2Config:
    hidden_size: int
    intermediate_size: int
    vocab_size: int
    num_hidden_layers: int = 5
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    block_size: int = 8
    conv_group_size: int = 16
    conv_kernel_size: int = 2
    mask_token_id: int = 0
    selector_rank: int = 256
    selector_top_k: int = 16
    sliding_window: int = 2048
    target_layer_ids: list[int] = field(default_factory=list)
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e7

    def __post_init__(self):
        assert self.hidden_size % self.conv_group_size == 0 and self.head_dim % 2 == 0
        assert self.num_attention_heads % self.num_key_value_heads == 0
        assert self.block_size >= 2 and 1 <= self.selector_top_k <= self.vocab_size and self.target_layer_ids

    @property
    def draft_tokens(self) -> int:
        return self.block_size - 1

    @property
    def conv_groups(self) -> int:
        return self.hidden_size // self.conv_group_size

    @staticmethod
    def from_json(path: str | Path) -> "QwenDFlash2Config":
        raw = json.loads(Path(path).read_text())
        df = raw.get("dflash_config", raw)
        rope = raw.get("rope_parameters", raw)
        if (raw.get("architectures") or [""])[0] != "DFlash2DraftModel":
            raise ValueError("not a DFlash2 drafter checkpoint")
        if raw.get("is_causal", False) or raw.get("attention_bias", False) or raw.get("hidden_act", "silu") != "silu" \
                or rope.get("rope_type", "default") != "default" \
                or any(t != "sliding_attention" for t in raw.get("layer_types", [])):
            raise ValueError("unsupported DFlash2 drafter semantics")
        return QwenDFlash2Config(
            hidden_size=raw["hidden_size"], intermediate_size=raw["intermediate_size"], vocab_size=raw["vocab_size"],
            num_hidden_layers=raw["num_hidden_layers"], num_attention_heads=raw["num_attention_heads"],
            num_key_value_heads=raw["num_key_value_heads"], head_dim=raw["head_dim"],
            block_size=df.get("block_size", raw.get("block_size", 0)), conv_group_size=df["conv_group_size"],
            conv_kernel_size=df["conv_kernel_size"], mask_token_id=df["mask_token_id"], selector_rank=df["selector_rank"],
            selector_top_k=df["selector_top_k"], sliding_window=raw["sliding_window"],
            target_layer_ids=list(df["target_layer_ids"]), rms_norm_eps=raw.get("rms_norm_eps", 1e-6),
            rope_theta=rope.get("rope_theta", 1e7))

    def to_json(self) -> dict:
        return {"architectures": ["DFlash2DraftModel"], "hidden_size": self.hidden_size,
                "intermediate_size": self.intermediate_size, "vocab_size": self.vocab_size,
                "num_hidden_layers": self.num_hidden_layers, "num_attention_heads": self.num_attention_heads,
                "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
                "sliding_window": self.sliding_window, "rms_norm_eps": self.rms_norm_eps, "hidden_act": "silu",
                "attention_bias": False, "is_causal": False, "num_target_layers": len(self.target_layer_ids),
                "layer_types": ["sliding_attention"] * self.num_hidden_layers,
                "rope_parameters": {"rope_type": "default", "rope_theta": self.rope_theta},
                "dflash_config": {"block_size": self.block_size, "conv_group_size": self.conv_group_size,
                                  "conv_kernel_size": self.conv_kernel_size, "mask_token_id": self.mask_token_id,
                                  "selector_rank": self.selector_rank, "selector_top_k": self.selector_top_k,
                                  "target_layer_ids": list(self.target_layer_ids)}}


def expected_tensors(cfg: QwenDFlash2Config) -> dict[str, tuple[int, ...]]:
    """Name -> shape of every tensor of a drafter checkpoint (6 global + 15 per layer)."""
    h, inter, d, kk, g = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim, cfg.conv_kernel_size, cfg.conv_groups
    qd, kvd = cfg.num_attention_heads * d, cfg.num_key_value_heads * d
    t = {"fc.weight": (h, h * len(cfg.target_layer_ids)), "hidden_norm.weight": (h,), "norm.weight": (h,),
         "candidate_selector.predecessor_codebook": (cfg.vocab_size, cfg.selector_rank),
         "candidate_selector.successor_codebook": (cfg.vocab_size, cfg.selector_rank),
         "candidate_selector.hidden_projection.weight": (cfg.selector_rank, h)}
    for i in range(cfg.num_hidden_layers):
        p = f"layers.{i}."
        t.update({p + "input_layernorm.weight": (h,), p + "post_attention_layernorm.weight": (h,),
                  p + "self_attn.q_proj.weight": (qd, h), p + "self_attn.k_proj.weight": (kvd, h),
                  p + "self_attn.v_proj.weight": (kvd, h), p + "self_attn.o_proj.weight": (h, qd),
                  p + "self_attn.q_norm.weight": (d,), p + "self_attn.k_norm.weight": (d,),
                  p + "mlp.gate_proj.weight": (inter, h), p + "mlp.up_proj.weight": (inter, h),
                  p + "mlp.down_proj.weight": (h, inter)})
        for c in ("attention_conv", "mlp_conv"):
            t[p + c + ".base_kernel"] = (2, kk, h)
            t[p + c + ".kernel_projection.weight"] = (2 * kk * g, h)
    return t


def synth_dflash2_weights(cfg: QwenDFlash2Config, seed: int = 0, std: float = 0.05) -> dict[str, torch.Tensor]:
    """Seeded random drafter in checkpoint dtype (bf16).  The base convolution kernels start near "pass the current
    row through" (tap 0 near 1, older taps small), as a trained drafter's do."""
    g = torch.Generator().manual_seed(seed + 1777)
    w = {}
    for name, shape in expected_tensors(cfg).items():
        if name.endswith(("norm.weight", "layernorm.weight")):
            t = 1.0 + torch.randn(*shape, generator=g) * 0.05
        elif name.endswith("base_kernel"):
            t = torch.randn(*shape, generator=g) * 0.1
            t[:, 0] += 1.0
        elif name.startswith("candidate_selector"):
            t = torch.randn(*shape, generator=g) * 0.5
        else:
            t = torch.randn(*shape, generator=g) * std
        w[name] = t.to(torch.bfloat16)
    return w


def load_dflash2(directory: str | Path) -> tuple[QwenDFlash2Config, dict[str, torch.Tensor]]:
    from ..formats import safetensors_io
    directory = Path(directory)
    cfg = QwenDFlash2Config.from_json(directory / "config.json")
    w = {k: v for k, v in safetensors_io.read_checkpoint(str(directory))}
    want = expected_tensors(cfg)
    missing, extra = sorted(set(want) - set(w)), sorted(set(w) - set(want))
    if missing or extra:
        raise ValueError(f"DFlash2 checkpoint does not hold exactly the expected {len(want)} tensors: "
                         f"missing {missing[:4]}, unexpected {extra[:4]}")
    for k, shape in want.items():
        if tuple(w[k].shape) != shape:
            raise ValueError(f"DFlash2 tensor {k}: shape {tuple(w[k].shape)}, expected {shape}")
    return cfg, w


def dynamic_conv(x: torch.Tensor, dyn: torch.Tensor, base: torch.Tensor, group_size: int) -> torch.Tensor:
    """x [rows, H]; dyn [rows, K * groups] (tap-major); base [K, H].  Causal over rows, zero history."""
    return sel.grouped_dynamic_conv(x, dyn, base, group_size)


def _rope_plain(x: torch.Tensor, start: int, theta: float) -> torch.Tensor:
    rows, half = x.shape[0], x.shape[-1] // 2
    inv = theta ** (-2.0 * torch.arange(half, dtype=torch.float32) / x.shape[-1])
    ang = (torch.arange(rows, dtype=torch.float32) + start)[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)


def top_candidates(logits: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Per row the ``k`` largest logits, best first; among equal logits the lower token id wins."""
    return sel.sharded_topk([logits], k)


def select_path(proj: torch.Tensor, cand: torch.Tensor, unary: torch.Tensor, pred: torch.Tensor, succ: torch.Tensor,
                anchor: int, viterbi: bool = False) -> list[int]:
    """proj [rows, rank]; cand / unary [rows, k]; pred / succ [vocab, rank].  One token per row: the greedy chain (each
    row conditioned on the previous pick, the anchor first) or the best whole path."""
    fn = sel.viterbi_path if viterbi else sel.greedy_path
    return fn(proj, cand, unary, pred, succ, anchor)[0]


@dataclass
class DFlash2Proposal:
    tokens: list[int]
    candidates: torch.Tensor            # [draft rows, k]
    candidate_logits: torch.Tensor


class QwenDFlash2Ref:
    def __init__(self, cfg: QwenDFlash2Config, weights: dict[str, torch.Tensor], embedding: torch.Tensor,
                 head: torch.Tensor, max_context: int = 4096, viterbi: bool = False, refine_passes: int = 1):
        self.cfg, self.max_context, self.viterbi, self.refine_passes = cfg, max_context, viterbi, max(1, refine_passes)
        self.w = {k: v.float() for k, v in weights.items()}
        self.embedding, self.head = embedding.float(), head.float()
        if self.embedding.shape != (cfg.vocab_size, cfg.hidden_size) or self.head.shape != self.embedding.shape:
            raise ValueError("DFlash2 drafter does not match the target's embedding / head")
        width = cfg.hidden_size * len(cfg.target_layer_ids)
        kvd = cfg.num_key_value_heads * cfg.head_dim
        self.taps = torch.zeros(max_context, width)
        self.ctx_k = [torch.zeros(max_context, kvd) for _ in range(cfg.num_hidden_layers)]
        self.ctx_v = [torch.zeros(max_context, kvd) for _ in range(cfg.num_hidden_layers)]
        self.committed = 0
        self.prepared = 0                      # rows whose keys and values are up to date
        self.debug = None                      # callable(name, tensor): every named stage of the next passes, as it is made
        self.context_begin = 0                 # first context row the block attends to (fixtures that start mid-sequence)

    def reset(self, begin: int = 0) -> None:
        """Empty context; ``begin`` > 0 starts it at that position (rows before it do not exist)."""
        self.committed = self.prepared = self.context_begin = begin

    def crop_context(self, position: int) -> None:
        if not 0 <= position <= self.committed:
            raise ValueError("invalid DFlash2 context crop")
        self.committed = position
        self.prepared = min(self.prepared, position)

    def append_target_taps(self, taps: torch.Tensor, position_offset: int) -> None:
        """Only stores the rows; keys and values are made when the next proposal needs them."""
        rows = taps.shape[0]
        if rows <= 0 or position_offset != self.committed or position_offset + rows > self.max_context \
                or taps.shape[1] != self.taps.shape[1]:
            raise ValueError("invalid DFlash2 target tap append")
        self.taps[position_offset:position_offset + rows] = taps.float()
        self.committed += rows

    def _tap(self, name: str, t) -> None:
        if self.debug is not None:
            self.debug(name, t if isinstance(t, torch.Tensor) else torch.tensor(t, dtype=torch.int32))

    @torch.no_grad()
    def _prepare_context(self) -> None:
        cfg, w, a, b = self.cfg, self.w, self.prepared, self.committed
        if a == b:
            return
        proj = self.taps[a:b] @ w["fc.weight"].t()
        ctx = _norm(proj, w["hidden_norm.weight"], cfg.rms_norm_eps)
        self._tap("context.projected", proj)
        self._tap("context.normalized", ctx)
        for i in range(cfg.num_hidden_layers):
            p, t = f"layers.{i}.self_attn.", f"layer.{i}.context."
            k = ctx @ w[p + "k_proj.weight"].t()
            v = ctx @ w[p + "v_proj.weight"].t()
            kn = _norm(k.view(b - a, cfg.num_key_value_heads, cfg.head_dim), w[p + "k_norm.weight"], cfg.rms_norm_eps)
            kr = _rope_plain(kn, a, cfg.rope_theta)
            for name, val in (("k_projection", k), ("v", v), ("k_norm", kn.reshape(b - a, -1)), ("k_rope", kr.reshape(b - a, -1))):
                self._tap(t + name, val)
            self.ctx_k[i][a:b] = kr.reshape(b - a, -1)
            self.ctx_v[i][a:b] = v
        self.prepared = b

    @torch.no_grad()
    def denoise(self, tokens: list[int]) -> torch.Tensor:
        """Final-normed hidden rows [block_size, hidden] for the block ``tokens`` (row 0 is the anchor)."""
        self._prepare_context()
        cfg, w, eps, n, tap = self.cfg, self.w, self.cfg.rms_norm_eps, self.committed, self._tap
        b, hq, hkv, d = cfg.block_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        kg, gs, win = cfg.conv_kernel_size * cfg.conv_groups, cfg.conv_group_size, cfg.sliding_window
        r = self.embedding[torch.tensor(tokens)]
        tap("noise.tokens", tokens)
        tap("noise.embedding", r)
        tap("residual.initial", r)
        lo = self.context_begin
        qpos = n + torch.arange(b)
        kpos = torch.cat([torch.arange(lo, n), qpos])
        mask = (qpos[:, None] - kpos[None, :]).abs() < win                  # [b, n - lo + b]
        for i in range(cfg.num_hidden_layers):
            p, t = f"layers.{i}.", f"layer.{i}."
            x = _norm(r, w[p + "input_layernorm.weight"], eps)
            dyn = x @ w[p + "attention_conv.kernel_projection.weight"].t()
            base = w[p + "attention_conv.base_kernel"]
            c = dynamic_conv(x, dyn[:, :kg], base[0], gs)
            tap(t + "input_norm", x); tap(t + "attention.dynamic", dyn); tap(t + "attention.prepare", c)
            q0, k0 = c @ w[p + "self_attn.q_proj.weight"].t(), c @ w[p + "self_attn.k_proj.weight"].t()
            v = (c @ w[p + "self_attn.v_proj.weight"].t()).view(b, hkv, d)
            q1 = _norm(q0.view(b, hq, d), w[p + "self_attn.q_norm.weight"], eps)
            k1 = _norm(k0.view(b, hkv, d), w[p + "self_attn.k_norm.weight"], eps)
            q, k = _rope_plain(q1, n, cfg.rope_theta), _rope_plain(k1, n, cfg.rope_theta)
            for name, val in (("q_projection", q0), ("k_projection", k0), ("v", v), ("q_norm", q1), ("k_norm", k1),
                              ("q_rope", q), ("k_rope", k)):
                tap(t + "attention." + name, val.reshape(b, -1))
            keys = torch.cat([self.ctx_k[i][lo:n].view(n - lo, hkv, d), k], 0).repeat_interleave(hq // hkv, 1)
            vals = torch.cat([self.ctx_v[i][lo:n].view(n - lo, hkv, d), v], 0).repeat_interleave(hq // hkv, 1)
            s = torch.einsum("qhd,khd->hqk", q, keys) / math.sqrt(d)
            s = s.masked_fill(~mask[None], float("-inf"))
            o = torch.einsum("hqk,khd->qhd", s.softmax(-1), vals).reshape(b, hq * d)
            op = o @ w[p + "self_attn.o_proj.weight"].t()
            fin = dynamic_conv(op, dyn[:, kg:], base[1], gs)
            r = r + fin
            tap(t + "attention.output", o); tap(t + "attention.o_projection", op); tap(t + "attention.finish", fin)
            tap(t + "attention.residual", r)
            x = _norm(r, w[p + "post_attention_layernorm.weight"], eps)
            dyn = x @ w[p + "mlp_conv.kernel_projection.weight"].t()
            base = w[p + "mlp_conv.base_kernel"]
            c = dynamic_conv(x, dyn[:, :kg], base[0], gs)
            gate, up = c @ w[p + "mlp.gate_proj.weight"].t(), c @ w[p + "mlp.up_proj.weight"].t()
            act = F.silu(gate) * up
            down = act @ w[p + "mlp.down_proj.weight"].t()
            fin = dynamic_conv(down, dyn[:, kg:], base[1], gs)
            r = r + fin
            for name, val in (("post_norm", x), ("mlp.dynamic", dyn), ("mlp.prepare", c), ("mlp.gate", gate), ("mlp.up", up),
                              ("mlp.swiglu", act), ("mlp.down", down), ("mlp.finish", fin), ("residual", r)):
                tap(t + name, val)
        out = _norm(r, w["norm.weight"], eps)
        tap("final.residual", r); tap("final.norm", out)
        return out

    @torch.no_grad()
    def _pass(self, anchor: int, tokens: list[int]) -> tuple[list[int], torch.Tensor, torch.Tensor]:
        cfg, w = self.cfg, self.w
        x = self.denoise(tokens)[1:]
        logits = x @ self.head.t()
        cand, unary = top_candidates(logits, cfg.selector_top_k)
        proj = x @ w["candidate_selector.hidden_projection.weight"].t()
        path = select_path(proj, cand, unary, w["candidate_selector.predecessor_codebook"],
                           w["candidate_selector.successor_codebook"], anchor, self.viterbi)
        self._tap("logits.local", logits)
        for scope in ("local", "global"):                       # one rank: the merged list is the local one
            self._tap(f"topk.{scope}.tokens", cand.to(torch.int32)); self._tap(f"topk.{scope}.logits", unary)
        self._tap("selector.path", path)
        return path, cand, unary

    @torch.no_grad()
    def propose(self, anchor: int) -> DFlash2Proposal:
        cfg = self.cfg
        if not 0 <= anchor < cfg.vocab_size or self.committed >= self.max_context:
            raise ValueError("invalid DFlash2 proposal anchor")
        self._prepare_context()
        tokens = [anchor] + [cfg.mask_token_id] * cfg.draft_tokens
        path, cand, unary = self._pass(anchor, tokens)
        for _ in range(1, self.refine_passes):
            nxt = [anchor] + path
            if nxt == tokens:
                break
            tokens = nxt
            path, cand, unary = self._pass(anchor, tokens)
        return DFlash2Proposal(path, cand, unary)


class QwenDFlash2Drafter:
    """The drafter behind the ``propose(context, k)`` protocol of ``components/speculative.py`` (see
    ``QwenDSparkDrafter``).  The confidence of a draft is the margin of its row's best candidate logit over the second."""

    def __init__(self, target, drafter: QwenDFlash2Ref):
        self.t, self.d = target, drafter
        target.oracle.capture_layers = tuple(drafter.cfg.target_layer_ids)

    def propose(self, context: list[int], k: int) -> tuple[list[int], list[float]]:
        taps = getattr(self.t, "taps", None)
        n = len(context) - 1
        if k <= 0 or taps is None or taps.shape[0] < n or n + self.d.cfg.block_size > self.d.max_context:
            return [], []
        if self.d.committed > n:
            self.d.reset()
        if self.d.committed < n:
            self.d.append_target_taps(taps[self.d.committed:n], self.d.committed)
        prop = self.d.propose(context[-1])
        u = prop.candidate_logits
        margin = (u[:, 0] - u[:, 1]).tolist() if u.shape[1] > 1 else [0.0] * u.shape[0]
        return prop.tokens[:k], margin[:k]
