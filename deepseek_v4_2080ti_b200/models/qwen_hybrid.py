"""Qwen-style hybrid runtime: Gated DeltaNet layers interleaved with gated full GQA attention.

Covers what the reference's native ``QwenEngine`` does (cpp_engine/engine/qwen_engine.cpp:
``run_chunk`` :4089-4269, ``layer_forward`` :3159-3313, ``linear_attention`` :2297-2540,
``full_attention`` :2544-3155): FP8 block-128 weights, bf16 activations, paged KV cache,
per-slot recurrent state, chunked prefill, batched decode, vocab-parallel embedding/head and
tensor-parallel sharding of heads and MLP.  Every op on the forward path is one of this
package's sm_100a kernels; decode steps are replayed from CUDA graphs.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Iterator

import torch

from ..formats import fp8 as fp8fmt
from ..utils import canary
from ..utils.phase_profile import PROFILER
from ..ops import _lib, attention, basic, gdn, gemm
from ..ops.gemm import PackedLinear


# ------------------------------------------------------------------ config
@dataclass
class QwenHybridConfig:
    vocab_size: int = 151936
    hidden_size: int = 5120
    intermediate_size: int = 17408
    num_hidden_layers: int = 64
    num_attention_heads: int = 40
    num_key_value_heads: int = 8
    head_dim: int = 128
    attn_output_gate: bool = True
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 32
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_conv_kernel_dim: int = 4
    max_position_embeddings: int = 262144
    rms_norm_eps: float = 1e-6
    partial_rotary_factor: float = 0.25
    rope_theta: float = 1e7
    full_attention_interval: int = 4
    layer_types: list[str] = field(default_factory=list)

    def __post_init__(self):
        if not self.layer_types:
            self.layer_types = [
                "full_attention" if (i + 1) % self.full_attention_interval == 0 else "linear_attention"
                for i in range(self.num_hidden_layers)
            ]
        assert len(self.layer_types) == self.num_hidden_layers
        assert self.head_dim == 128 and self.linear_key_head_dim == 128 and self.linear_value_head_dim == 128, \
            "kernels are specialised for 128-wide heads"

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    @staticmethod
    def from_json(path: str | Path) -> "QwenHybridConfig":
        """HF-style config.json (``Qwen3_5ForConditionalGeneration`` with ``text_config``), as parsed by
        cpp_engine/core/qwen_config.cpp:150-240."""
        raw = json.loads(Path(path).read_text())
        tc = raw.get("text_config", raw)
        rp = tc.get("rope_parameters", {}) or {}
        known = {f for f in QwenHybridConfig.__dataclass_fields__}
        kw = {k: v for k, v in tc.items() if k in known}
        if "rope_theta" in rp:
            kw["rope_theta"] = float(rp["rope_theta"])
        if "partial_rotary_factor" in rp:
            kw["partial_rotary_factor"] = float(rp["partial_rotary_factor"])
        return QwenHybridConfig(**kw)

    def to_json(self) -> str:
        tc = {k: getattr(self, k) for k in self.__dataclass_fields__ if k not in ("rope_theta", "full_attention_interval")}
        tc["model_type"] = "qwen3_5_text"
        tc["rope_parameters"] = {"rope_type": "default", "rope_theta": self.rope_theta}
        return json.dumps({"architectures": ["Qwen3_5ForConditionalGeneration"], "model_type": "qwen3_5",
                           "text_config": tc}, indent=1)

    @staticmethod
    def config2() -> "QwenHybridConfig":
        """The 27B-class benchmark shape: 64 layers, hidden 5120, 48 GDN + 16 gated-GQA layers."""
        return QwenHybridConfig()

    @staticmethod
    def tiny(layers: int = 4, hidden: int = 256, vocab: int = 512) -> "QwenHybridConfig":
        return QwenHybridConfig(vocab_size=vocab, hidden_size=hidden, intermediate_size=384, num_hidden_layers=layers,
                                num_attention_heads=4, num_key_value_heads=2, linear_num_key_heads=2,
                                linear_num_value_heads=4, max_position_embeddings=8192, full_attention_interval=2)


# ------------------------------------------------------- synthetic checkpoints
FP8_SUFFIXES = ("in_proj_qkv", "in_proj_z", "out_proj", "q_proj", "k_proj", "v_proj", "o_proj", "gate_proj",
                "up_proj", "down_proj")


def tensor_specs(cfg: QwenHybridConfig) -> list[tuple[str, tuple[int, ...], str]]:
    """(name, shape, kind) for every checkpoint tensor, in the reference's naming
    (cpp_engine/tests/qwen_parity_fixture.hpp:117-170). kind: fp8 | bf16 | norm | a_log | dt_bias."""
    h, inter = cfg.hidden_size, cfg.intermediate_size
    kd = cfg.linear_num_key_heads * cfg.linear_key_head_dim
    vd = cfg.linear_num_value_heads * cfg.linear_value_head_dim
    hv = cfg.linear_num_value_heads
    qd = cfg.num_attention_heads * cfg.head_dim
    kvd = cfg.num_key_value_heads * cfg.head_dim
    out: list[tuple[str, tuple[int, ...], str]] = [
        ("model.language_model.embed_tokens.weight", (cfg.vocab_size, h), "bf16"),
        ("model.language_model.norm.weight", (h,), "norm"),
        ("lm_head.weight", (cfg.vocab_size, h), "bf16"),
    ]
    for i, lt in enumerate(cfg.layer_types):
        p = f"model.language_model.layers.{i}."
        out += [(p + "input_layernorm.weight", (h,), "norm"), (p + "post_attention_layernorm.weight", (h,), "norm")]
        if lt == "linear_attention":
            a = p + "linear_attn."
            out += [(a + "in_proj_qkv.weight", (2 * kd + vd, h), "fp8"), (a + "in_proj_z.weight", (vd, h), "fp8"),
                    (a + "out_proj.weight", (h, vd), "fp8"), (a + "in_proj_a.weight", (hv, h), "bf16"),
                    (a + "in_proj_b.weight", (hv, h), "bf16"), (a + "conv1d.weight", (2 * kd + vd, 1, cfg.linear_conv_kernel_dim), "conv"),
                    (a + "A_log", (hv,), "a_log"), (a + "dt_bias", (hv,), "dt_bias"),
                    (a + "norm.weight", (cfg.linear_value_head_dim,), "norm1")]
        else:
            a = p + "self_attn."
            q_out = qd * (2 if cfg.attn_output_gate else 1)
            out += [(a + "q_proj.weight", (q_out, h), "fp8"), (a + "k_proj.weight", (kvd, h), "fp8"),
                    (a + "v_proj.weight", (kvd, h), "fp8"), (a + "o_proj.weight", (h, qd), "fp8"),
                    (a + "q_norm.weight", (cfg.head_dim,), "norm"), (a + "k_norm.weight", (cfg.head_dim,), "norm")]
        m = p + "mlp."
        out += [(m + "gate_proj.weight", (inter, h), "fp8"), (m + "up_proj.weight", (inter, h), "fp8"),
                (m + "down_proj.weight", (h, inter), "fp8")]
    return out


def synth_state(cfg: QwenHybridConfig, seed: int = 0, device: str | torch.device = "cpu",
                std: float = 0.02) -> Iterator[tuple[str, torch.Tensor]]:
    """Seeded random-init checkpoint tensors in checkpoint dtypes: N(0, std) weights quantised to
    FP8 E4M3 with bf16 128x128 ``weight_scale_inv``; (1+gamma) norms near 0; plain norms near 1."""
    gen = torch.Generator(device=device)
    for idx, (name, shape, kind) in enumerate(tensor_specs(cfg)):
        gen.manual_seed(seed * 1_000_003 + idx)
        if kind == "fp8":
            w = torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std
            q, s = fp8fmt.quantize_block128(w)
            del w
            yield name, q
            yield name + "_scale_inv", s
        elif kind == "bf16":
            yield name, (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std).bfloat16()
        elif kind == "conv":
            yield name, (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * 0.3).bfloat16()
        elif kind == "norm":
            yield name, (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * 0.05).bfloat16()
        elif kind == "norm1":
            yield name, (1.0 + torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * 0.05).bfloat16()
        elif kind == "a_log":
            yield name, torch.log(torch.rand(shape, generator=gen, device=device) * 3.0 + 0.5).bfloat16()
        elif kind == "dt_bias":
            yield name, (torch.rand(shape, generator=gen, device=device) * 2.0 - 1.0).bfloat16()
        else:
            raise ValueError(kind)


# ------------------------------------------------------------------ weights
def _shard_rows(t: torch.Tensor, rank: int, world: int, group: int = 1) -> torch.Tensor:
    n = t.shape[0] // world
    assert n * world == t.shape[0] and n % group == 0
    return t[rank * n:(rank + 1) * n]


def _shard_scale_rows(s: torch.Tensor, rows: int, rank: int, world: int) -> torch.Tensor:
    n = rows // world
    assert n % 128 == 0 or world == 1, "TP shard of an FP8 matrix must keep whole 128-row scale blocks"
    return s[rank * n // 128:(rank * n + n + 127) // 128]


@dataclass
class LayerWeights:
    kind: str
    in_ln: torch.Tensor
    post_ln: torch.Tensor
    proj: PackedLinear            # linear: qkv|z ; full: q(|gate)|k|v
    out: PackedLinear             # out_proj / o_proj (row-parallel)
    gate_up: PackedLinear
    down: PackedLinear            # row-parallel
    ab: PackedLinear | None = None
    conv_w: torch.Tensor | None = None
    a_log: torch.Tensor | None = None
    dt_bias: torch.Tensor | None = None
    gdn_norm: torch.Tensor | None = None
    q_norm: torch.Tensor | None = None
    k_norm: torch.Tensor | None = None


@dataclass
class MtpWeights:
    norm_embed: torch.Tensor
    norm_hidden: torch.Tensor
    norm_out: torch.Tensor
    fc: PackedLinear              # [H, 2H], replicated
    layer: LayerWeights           # one full-attention decoder layer


class QwenHybridWeights:
    """Device-resident, TP-sharded, kernel-ready weights built from (name, tensor) pairs."""

    def __init__(self, cfg: QwenHybridConfig, state: Iterator[tuple[str, torch.Tensor]], device, tp_rank: int = 0,
                 tp_world: int = 1, replicate_embedding: bool = True):
        """``replicate_embedding``: every rank keeps the whole embedding table (1.5 GB at the 27B shape, nothing
        against 180 GB), so the lookup needs no collective; False gives the vocabulary-parallel table with a masked
        lookup + all-reduce, as the reference does on 22 GB cards (cpp_engine/engine/qwen_engine.cpp:4113-4118).
        The output head is vocabulary-parallel either way."""
        self.cfg, self.device, self.rank, self.world = cfg, torch.device(device), tp_rank, tp_world
        self.embed_replicated = bool(replicate_embedding) or tp_world == 1
        self.layers: list[LayerWeights | None] = [None] * cfg.num_hidden_layers
        self._pending: dict[str, torch.Tensor] = {}
        self.embed = self.lm_head = self.final_norm = None
        self.vocab_lo = self.vocab_hi = 0
        for name, t in state:
            self._pending[name] = t
            self._try_finish(name)
        missing = [i for i, l in enumerate(self.layers) if l is None]
        if missing or self.embed is None or self.lm_head is None or self.final_norm is None:
            raise ValueError(f"checkpoint incomplete: layers {missing[:4]}... pending {list(self._pending)[:6]}")
        self.mtp = self._build_mtp()

    # -- helpers
    def _dev(self, t):
        return t.to(self.device, non_blocking=True)

    def _fp8(self, base: str):
        return self._pending.pop(base + ".weight"), self._pending.pop(base + ".weight_scale_inv")

    def _nvfp4(self, base: str) -> torch.Tensor:
        """bf16 [N, K] on the device from the three NVFP4 tensors of ``base``."""
        from ..formats import nvfp4
        P = self._pending
        return nvfp4.dequantize(self._dev(P.pop(base + ".weight_packed")), self._dev(P.pop(base + ".weight_scale")),
                                self._dev(P.pop(base + ".weight_global_scale")), torch.bfloat16)

    def _col_fp8(self, parts: list[tuple[torch.Tensor, torch.Tensor, int]]) -> PackedLinear:
        """Concatenate column-parallel FP8 pieces (each already row-sharded) along N."""
        ws, ss = [], []
        for w, s, rows_total in parts:
            ws.append(self._dev(w))
            ss.append(self._dev(s))
        w = torch.cat(ws, 0) if len(ws) > 1 else ws[0]
        s = torch.cat(ss, 0) if len(ss) > 1 else ss[0]
        return PackedLinear.from_fp8(w.contiguous(), s.contiguous())

    def _rows_fp8(self, w, s, group_rows: int | None = None):
        """Row (output-feature) shard of an FP8 matrix + its scale rows."""
        if self.world == 1:
            return w, s, w.shape[0]
        n = w.shape[0] // self.world
        assert n % 128 == 0, f"TP row shard {n} is not a multiple of the 128-row scale block"
        r = self.rank
        return w[r * n:(r + 1) * n], s[r * n // 128:(r + 1) * n // 128], w.shape[0]

    def _cols_fp8(self, w, s) -> PackedLinear:
        """Column (input-feature) shard for row-parallel matrices."""
        if self.world > 1:
            k = w.shape[1] // self.world
            assert k % 128 == 0
            r = self.rank
            w, s = w[:, r * k:(r + 1) * k], s[:, r * k // 128:(r + 1) * k // 128]
        return PackedLinear.from_fp8(self._dev(w).contiguous(), self._dev(s).contiguous())

    def _try_finish(self, name: str) -> None:
        cfg, P = self.cfg, self._pending
        if name == "model.language_model.embed_tokens.weight":
            t = P.pop(name)
            n = (cfg.vocab_size + self.world - 1) // self.world
            self.vocab_lo, self.vocab_hi = self.rank * n, min(cfg.vocab_size, (self.rank + 1) * n)
            if self.embed_replicated:
                self.vocab_lo, self.vocab_hi = 0, cfg.vocab_size
            self.embed = self._dev(t[self.vocab_lo:self.vocab_hi]).contiguous()
            return
        if name == "lm_head.weight":
            t = P.pop(name)
            n = (cfg.vocab_size + self.world - 1) // self.world
            lo, hi = self.rank * n, min(cfg.vocab_size, (self.rank + 1) * n)
            self.lm_head = PackedLinear.from_bf16(self._dev(t[lo:hi]))
            self.head_lo = lo
            return
        if name == "model.language_model.norm.weight":
            self.final_norm = self._dev(P.pop(name))
            return
        if not name.startswith("model.language_model.layers."):
            return
        i = int(name.split(".")[3])
        if self.layers[i] is not None:
            return
        lw = self._build_layer(f"model.language_model.layers.{i}.", cfg.layer_types[i])
        if lw is not None:
            self.layers[i] = lw

    def _build_layer(self, p: str, lt: str) -> "LayerWeights | None":
        """Kernel-ready, TP-sharded weights of the decoder layer whose tensors start with ``p``, once all of them
        have arrived (None before that)."""
        cfg, P = self.cfg, self._pending
        need = [p + "input_layernorm.weight", p + "post_attention_layernorm.weight"]
        nvfp4_mlp = (p + "mlp.gate_proj.weight_packed") in P or (p + "mlp.gate_proj.weight_scale") in P or \
            (p + "mlp.gate_proj.weight_global_scale") in P
        for m in ("gate_proj", "up_proj", "down_proj"):
            if nvfp4_mlp:
                need += [p + f"mlp.{m}.weight_packed", p + f"mlp.{m}.weight_scale", p + f"mlp.{m}.weight_global_scale"]
            else:
                need += [p + f"mlp.{m}.weight", p + f"mlp.{m}.weight_scale_inv"]
        if lt == "linear_attention":
            a = p + "linear_attn."
            for m in ("in_proj_qkv", "in_proj_z", "out_proj"):
                need += [a + m + ".weight", a + m + ".weight_scale_inv"]
            need += [a + "in_proj_a.weight", a + "in_proj_b.weight", a + "conv1d.weight", a + "A_log", a + "dt_bias",
                     a + "norm.weight"]
        else:
            a = p + "self_attn."
            for m in ("q_proj", "k_proj", "v_proj", "o_proj"):
                need += [a + m + ".weight", a + m + ".weight_scale_inv"]
            need += [a + "q_norm.weight", a + "k_norm.weight"]
        if not all(n in P for n in need):
            return None
        W, R = self.world, self.rank
        in_ln, post_ln = self._dev(P.pop(need[0])), self._dev(P.pop(need[1]))
        if nvfp4_mlp:
            # NVFP4 feed-forward matrices (mixed checkpoints keep FP8 elsewhere): expanded to bf16 once, sharded like
            # the FP8 ones, multiplied on the bf16 tile path
            g, u, d = (self._nvfp4(p + f"mlp.{m}") for m in ("gate_proj", "up_proj", "down_proj"))
            gate_up = PackedLinear.from_bf16(torch.cat([_shard_rows(g, R, W), _shard_rows(u, R, W)], 0))
            kk = d.shape[1] // W
            down = PackedLinear.from_bf16(d[:, R * kk:(R + 1) * kk])
            for m in ("gate_proj", "up_proj", "down_proj"):
                P.pop(p + f"mlp.{m}.input_global_scale", None)     # activations stay bf16 here
        else:
            g = self._rows_fp8(*self._fp8(p + "mlp.gate_proj"))
            u = self._rows_fp8(*self._fp8(p + "mlp.up_proj"))
            gate_up = self._col_fp8([g, u])
            down = self._cols_fp8(*self._fp8(p + "mlp.down_proj"))
        if lt == "linear_attention":
            a = p + "linear_attn."
            kd = cfg.linear_num_key_heads * 128
            vd = cfg.linear_num_value_heads * 128
            wq, sq = self._fp8(a + "in_proj_qkv")
            pieces = []
            conv = P.pop(a + "conv1d.weight").reshape(2 * kd + vd, -1)
            conv_parts = []
            for lo, n in ((0, kd), (kd, kd), (2 * kd, vd)):
                per = n // W
                assert per % 128 == 0
                pieces.append((wq[lo + R * per:lo + (R + 1) * per], sq[(lo + R * per) // 128:(lo + (R + 1) * per) // 128], n))
                conv_parts.append(conv[lo + R * per:lo + (R + 1) * per])
            pieces.append(self._rows_fp8(*self._fp8(a + "in_proj_z")))
            proj = self._col_fp8(pieces)
            out = self._cols_fp8(*self._fp8(a + "out_proj"))
            hv = cfg.linear_num_value_heads // W
            wa = _shard_rows(P.pop(a + "in_proj_a.weight"), R, W)
            wb = _shard_rows(P.pop(a + "in_proj_b.weight"), R, W)
            ab = PackedLinear.from_bf16(self._dev(torch.cat([wa, wb], 0)))
            assert hv * W == cfg.linear_num_value_heads
            return LayerWeights(
                "linear", in_ln, post_ln, proj, out, gate_up, down, ab=ab,
                conv_w=self._dev(torch.cat(conv_parts, 0)).contiguous(),
                a_log=self._dev(_shard_rows(P.pop(a + "A_log"), R, W)).float().contiguous(),
                dt_bias=self._dev(_shard_rows(P.pop(a + "dt_bias"), R, W)).float().contiguous(),
                gdn_norm=self._dev(P.pop(a + "norm.weight")))
        else:
            a = p + "self_attn."
            pieces = [self._rows_fp8(*self._fp8(a + "q_proj")), self._rows_fp8(*self._fp8(a + "k_proj")),
                      self._rows_fp8(*self._fp8(a + "v_proj"))]
            proj = self._col_fp8(pieces)
            out = self._cols_fp8(*self._fp8(a + "o_proj"))
            return LayerWeights("full", in_ln, post_ln, proj, out, gate_up, down,
                                q_norm=self._dev(P.pop(a + "q_norm.weight")),
                                k_norm=self._dev(P.pop(a + "k_norm.weight")))

    def _build_mtp(self) -> "MtpWeights | None":
        """The multi-token-prediction head, when the checkpoint carries one (``mtp.*``: two input norms, ``mtp.fc``
        [H, 2H], one full-attention decoder layer, ``mtp.norm``; embedding and output head are the trunk's).
        ``mtp.fc`` and the norms are replicated, the layer is sharded like the trunk's (cpp_engine/core/
        qwen_weight_map.cpp maps the same names; a checkpoint with some but not all of them is refused)."""
        P = self._pending
        if not any(k.startswith("mtp.") for k in P):
            return None
        # a head stored in bf16 is quantised to the trunk's FP8 block-128 format here, so its layer runs through the
        # same kernels (drafts only steer which tokens get verified; the verified output does not depend on them)
        for k in [k for k in P if k.startswith("mtp.layers.0.") and k.endswith("_proj.weight")]:
            if P[k].dtype != torch.float8_e4m3fn and (k + "_scale_inv") not in P:
                q, sc = fp8fmt.quantize_block128(P[k].to(self.device, torch.float32))
                P[k], P[k + "_scale_inv"] = q, sc
        layer = self._build_layer("mtp.layers.0.", "full_attention")
        names = ["mtp.pre_fc_norm_embedding.weight", "mtp.pre_fc_norm_hidden.weight", "mtp.norm.weight", "mtp.fc.weight"]
        if layer is None or not all(n in P for n in names):
            raise ValueError("checkpoint carries an incomplete multi-token-prediction head: "
                             f"{sorted(k for k in P if k.startswith('mtp.'))[:6]}")
        fc_w = P.pop("mtp.fc.weight")
        if fc_w.dtype == torch.float8_e4m3fn:
            fc = PackedLinear.from_fp8(self._dev(fc_w).contiguous(), self._dev(P.pop("mtp.fc.weight_scale_inv")).contiguous())
        else:
            fc = PackedLinear.from_bf16(self._dev(fc_w))
        return MtpWeights(self._dev(P.pop(names[0])), self._dev(P.pop(names[1])), self._dev(P.pop(names[2])), fc, layer)

    def nbytes(self) -> int:
        n = self.embed.numel() * 2 + self.lm_head.nbytes()
        for l in self.layers:
            n += l.proj.nbytes() + l.out.nbytes() + l.gate_up.nbytes() + l.down.nbytes()
            if l.ab is not None:
                n += l.ab.nbytes()
        return n


# ------------------------------------------------------------------ runtime
class NoComm:
    """Single-rank stand-in for the tensor-parallel communicator."""
    world, rank = 1, 0

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        return t

    def argmax_merge(self, idx: torch.Tensor, val: torch.Tensor) -> torch.Tensor:
        return idx

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        return t.unsqueeze(0)


@dataclass
class SeqState:
    slot: int
    blocks: list[int] = field(default_factory=list)
    length: int = 0


class QwenHybridRuntime:
    """Owns weights, the paged KV pool, per-slot recurrent state and the forward passes."""

    def __init__(self, cfg: QwenHybridConfig, weights: QwenHybridWeights, max_slots: int = 1,
                 max_context: int = 8192 + 512, block_size: int = 64, comm=None, num_blocks: int | None = None,
                 attention_window: int = 0, attention_sink_tokens: int = 0, kv_cache_dtype: str = "bf16"):
        """``attention_window`` > 0 restricts the full-attention layers to a sliding window of that many keys plus
        the first ``attention_sink_tokens`` keys (the cache still holds every position).  ``kv_cache_dtype`` "fp8",
        "int8_per_token_head" or "turboquant_k8v4" keeps the cache as E4M3 / INT8 rows (K8V4: E4M3 keys, 4-bit
        values) with one scale per (token, head): half (three eighths) of the bytes per token, read directly by the
        decode kernel and staged back to bf16 per layer for the prefill kernel."""
        if kv_cache_dtype not in ("auto", "bf16", "fp16", *attention.KV8_FORMATS):
            raise ValueError(f"unknown KV cache dtype {kv_cache_dtype!r}")
        self.kv_cache_dtype = kv_cache_dtype if kv_cache_dtype in attention.KV8_FORMATS else "bf16"
        self.cfg, self.w, self.device = cfg, weights, weights.device
        self.attention_window, self.attention_sinks = int(attention_window), int(attention_sink_tokens)
        self.comm = comm or NoComm()
        # prefill GEMMs in launch order: while one runs, the FP8 -> bf16 expansion of the next runs on a side stream
        chain = [m for lw in weights.layers for m in (lw.proj, lw.out, lw.gate_up, lw.down)]
        self._next_w = {id(a): b for a, b in zip(chain, chain[1:])}
        self._gate_up_ids = {id(lw.gate_up) for lw in weights.layers}
        W = self.comm.world
        assert W == weights.world
        self.hq = cfg.num_attention_heads // W
        self.hkv = max(1, cfg.num_key_value_heads // W)
        assert cfg.num_key_value_heads % W == 0, "kv heads must divide over the TP group"
        self.hk_lin = cfg.linear_num_key_heads // W
        self.hv_lin = cfg.linear_num_value_heads // W
        self.kd, self.vd = self.hk_lin * 128, self.hv_lin * 128
        self.block_size = block_size
        self.max_slots = max_slots
        self.max_blocks_per_seq = (max_context + block_size - 1) // block_size
        self.num_blocks = num_blocks or (self.max_blocks_per_seq * max_slots + 1)
        self.full_layers = [i for i, t in enumerate(cfg.layer_types) if t == "full_attention"]
        self.lin_layers = [i for i, t in enumerate(cfg.layer_types) if t == "linear_attention"]
        dev = self.device
        nf, nl = len(self.full_layers), len(self.lin_layers)
        self.mtp = getattr(weights, "mtp", None)
        if self.mtp is not None:
            nf += 1            # the head's attention layer keeps its keys/values as one more cache layer (index nf - 1)
        self.keep_hidden = False   # a speculator sets it: prefill then keeps the final-normed hidden of every row
        self.hidden_rows = None
        # block 0 is a scratch block: padded rows of a decode batch write their K/V there
        self.kv8 = None
        if self.kv_cache_dtype != "bf16":
            self.kv8 = attention.Kv8Cache(self.kv_cache_dtype, nf, self.num_blocks, self.hkv, block_size, dev)
            self.k_cache = self.v_cache = None
            # bf16 staging: one sequence's whole context for prefill (blocks in sequence order), one row per sequence
            # of a decode batch
            self.stage_k = torch.zeros(self.max_blocks_per_seq, self.hkv, block_size, 128, dtype=torch.bfloat16, device=dev)
            self.stage_v = torch.zeros_like(self.stage_k)
            drows = max(max_slots, 64)
            self.dstage_k = torch.zeros((drows + block_size - 1) // block_size, self.hkv, block_size, 128,
                                        dtype=torch.bfloat16, device=dev)
            self.dstage_v = torch.zeros_like(self.dstage_k)
            self._ident_bt = torch.arange(self.max_blocks_per_seq, dtype=torch.int32, device=dev)[None]
            self._rows = torch.arange(drows, dtype=torch.int32, device=dev)
        else:
            self.k_cache = canary.zeros(nf, self.num_blocks, self.hkv, block_size, 128, dtype=torch.bfloat16, device=dev,
                                        name="paged key cache")
            self.v_cache = canary.zeros(nf, self.num_blocks, self.hkv, block_size, 128, dtype=torch.bfloat16, device=dev,
                                        name="paged value cache")
        self.states = canary.zeros(max_slots, nl, self.hv_lin, 128, 128, dtype=torch.float32, device=dev,
                                   name="gated delta-net states")
        self.tails = torch.zeros(max_slots, nl, cfg.linear_conv_kernel_dim - 1, 2 * self.kd + self.vd,
                                 dtype=torch.bfloat16, device=dev)
        self.inv_freq = attention.rope_inv_freq(cfg.rotary_dim, cfg.rope_theta, dev)
        self.free_blocks = list(range(self.num_blocks - 1, 0, -1))
        self.block_refs = [0] * self.num_blocks        # sequences + prefix-cache entries holding each block
        self.prefix_cache = None
        self.prefill_tokens_computed = 0               # prompt tokens actually run through the model (cache hits skip)
        self.free_slots = list(range(max_slots - 1, -1, -1))
        self.seqs: dict[int, SeqState] = {}
        self.block_table = torch.zeros(max_slots, self.max_blocks_per_seq, dtype=torch.int32, device=dev)
        self._bt_host = torch.zeros(max_slots, self.max_blocks_per_seq, dtype=torch.int32)
        self._graphs: dict[int, tuple] = {}
        self.launches = 0  # kernels launched by the last forward (for the bench record)
        self._sp = False   # set while a sequence-parallel prefill chunk is in flight
        # decode batches of <= 32 rows take the fused path; needs every FP8 K dimension to be a multiple of 128
        from ..ops.gemm import WF_FP8_B128
        self.fused_decode = all(l.proj.k % 128 == 0 and l.out.k % 128 == 0 and l.down.k % 128 == 0 and
                                l.gate_up.k % 128 == 0 and l.gate_up.wfmt == WF_FP8_B128 and l.down.wfmt == WF_FP8_B128
                                for l in weights.layers) and \
            (self.hv_lin // max(1, self.hk_lin)) in (1, 2, 4) and cfg.linear_conv_kernel_dim == 4

    # ---- slot / block management (host side)
    def allocate(self) -> int:
        slot = self.free_slots.pop()
        self.seqs[slot] = SeqState(slot)
        self.states[slot].zero_()
        self.tails[slot].zero_()
        return slot

    def free(self, slot: int) -> None:
        st = self.seqs.pop(slot)
        self._release_blocks(st.blocks)
        self.free_slots.append(slot)

    def _release_blocks(self, blocks: list[int]) -> None:
        for b in reversed(blocks):
            self.block_refs[b] -= 1
            if self.block_refs[b] == 0:
                self.free_blocks.append(b)

    def enable_prefix_cache(self, interval: int = 256, max_entries: int = 8, max_bytes: int = 8 << 30):
        """Re-use KV blocks and recurrent-state snapshots of already-seen prompt prefixes (runtime/prefix_cache.py).
        ``interval`` (tokens between snapshot points) must be a multiple of the KV block size."""
        from ..runtime.prefix_cache import PrefixCache
        if interval % self.block_size:
            raise ValueError("snapshot interval must be a multiple of the KV block size")
        self.prefix_cache = PrefixCache(interval, max_entries, max_bytes, release_blocks=self._release_blocks)
        return self.prefix_cache

    def _restore_prefix(self, st: SeqState, tokens: list[int]) -> None:
        e = self.prefix_cache.lookup(tokens)
        if e is None:
            return
        for i, b in enumerate(e.blocks):
            self.block_refs[b] += 1
            self._bt_host[st.slot, i] = b
        st.blocks = list(e.blocks)
        self.block_table[st.slot].copy_(self._bt_host[st.slot], non_blocking=True)
        self.states[st.slot].copy_(e.snapshot[0])
        self.tails[st.slot].copy_(e.snapshot[1])
        st.length = e.tokens

    def _snapshot_prefix(self, st: SeqState, tokens: list[int]) -> None:
        n = st.length
        if self.prefix_cache.contains(tokens, n):
            return
        snap = (self.states[st.slot].clone(), self.tails[st.slot].clone())
        blocks = st.blocks[:n // self.block_size]
        nbytes = snap[0].numel() * 4 + snap[1].numel() * 2
        if self.prefix_cache.insert(tokens, n, blocks, snap, nbytes):
            for b in blocks:
                self.block_refs[b] += 1

    def _ensure_blocks(self, st: SeqState, new_len: int) -> None:
        need = (new_len + self.block_size - 1) // self.block_size
        if need > self.max_blocks_per_seq:
            raise RuntimeError("sequence exceeds max_context")
        changed = False
        while len(st.blocks) < need:
            if not self.free_blocks:
                raise RuntimeError("KV cache exhausted")
            b = self.free_blocks.pop()
            self.block_refs[b] = 1
            self._bt_host[st.slot, len(st.blocks)] = b
            st.blocks.append(b)
            changed = True
        if changed:
            self.block_table[st.slot].copy_(self._bt_host[st.slot], non_blocking=True)

    def recover_collectives(self) -> None:
        """After a collective timed out: re-synchronise the communicator (all ranks call this) and drop the captured
        decode graphs, which still hold the peer-memory kernels."""
        rec = getattr(self.comm, "recover", None)
        if rec is not None:
            rec()
        self._graphs.clear()

    # ---- layer bodies
    def _col_parallel(self, x: torch.Tensor, w: PackedLinear) -> torch.Tensor:
        """Column-parallel projection of the normalised activations.  Sequence-parallel chunks read the gathered
        buffer, whose rows arrive from the ranks that own them (all-gather + GEMM in one kernel)."""
        self._expand_ahead(x, w)
        if self._sp:
            return self.comm.linear_ag(x, w)
        return gemm.linear(x, w)

    def _expand_ahead(self, x: torch.Tensor, w: PackedLinear) -> None:
        if x.shape[0] >= gemm.PREDECODE_MIN_T:
            nxt = self._next_w.get(id(w))
            fused = nxt is not None and id(nxt) in self._gate_up_ids and self._swiglu_fused(x.shape[0], nxt)
            gemm.prefetch_bf16(nxt, x.device, w, gate_up=fused)

    def _swiglu_fused(self, t: int, w: PackedLinear) -> bool:
        """Does the feed-forward block of a ``t``-token chunk take the GEMM with the SwiGLU epilogue?  In a
        sequence-parallel chunk every rank's rows must also be whole 256-token tiles of that kernel."""
        if not gemm.swiglu_fusable(t, w):
            return False
        return not self._sp or (hasattr(self.comm, "linear_ag_swiglu") and (t // self.comm.world) % 256 == 0)

    def _row_parallel(self, x: torch.Tensor, w: PackedLinear) -> torch.Tensor | None:
        """Row-parallel projection: this rank's K-shard GEMM + sum over ranks.  With a peer-memory communicator the
        reduction happens in the GEMM epilogue (tile by tile over NVLink); otherwise GEMM then all-reduce.
        Sequence-parallel chunks only push the partial tiles to the owners of the rows (nothing is returned: the
        owner's reduce + norm + gather kernel picks them up)."""
        if self._sp:
            self._expand_ahead(x, w)
            self.comm.linear_rs(x, w)
            return None
        fused = getattr(self.comm, "linear_allreduce", None)
        if fused is not None and self.comm.world > 1:
            return fused(x, w)
        self._expand_ahead(x, w)
        return self.comm.all_reduce(gemm.linear(x, w))

    def _stream_row_parallel(self, x: torch.Tensor | None, w: PackedLinear, xsplit=None) -> torch.Tensor:
        """Row-parallel projection of a decode step (T <= 32): with a peer-memory communicator the all-reduce is done
        in the epilogue of the weight-streaming GEMM, otherwise GEMM then all-reduce."""
        fused = getattr(self.comm, "stream_allreduce", None)
        if fused is not None and self.comm.world > 1:
            return fused(x, w, xsplit=xsplit)
        return self.comm.all_reduce(gemm.linear_stream(x, w, xsplit=xsplit))

    def _mlp(self, lw: LayerWeights, h: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        if self._sp:
            x = self.comm.reduce_norm_gather(h, lw.post_ln, cfg.rms_norm_eps, True)
        else:
            x = basic.add_rmsnorm(h, delta, lw.post_ln, cfg.rms_norm_eps, True)
        with PROFILER.scope("lin.gate_up"):
            if self._swiglu_fused(x.shape[0], lw.gate_up):
                self._expand_ahead(x, lw.gate_up)
                act = self.comm.linear_ag_swiglu(x, lw.gate_up) if self._sp else gemm.linear_swiglu(x, lw.gate_up)
            else:
                act = basic.silu_mul(self._col_parallel(x, lw.gate_up))
        with PROFILER.scope("lin.down+ar.mlp"):
            return self._row_parallel(act, lw.down)

    def _linear_attn(self, li: int, lw: LayerWeights, x: torch.Tensor, t: int, slots_t: torch.Tensor | None,
                     slot: int | None) -> torch.Tensor:
        cfg = self.cfg
        with PROFILER.scope("lin.qkvz"):
            proj = self._col_parallel(x, lw.proj)            # [T, 2kd + vd + vd]
        ab = gemm.linear(x, lw.ab)                           # [T, 2 hv]
        cw = 2 * self.kd + self.vd
        idx = self.lin_layers.index(li)
        g, beta = basic.gdn_gates(ab, 0, self.hv_lin, lw.a_log, lw.dt_bias, self.hv_lin)
        if slot is not None:   # one sequence, T consecutive tokens
            mixed = basic.conv_silu(proj[:, :cw], lw.conv_w, self.tails[slot, idx])
            with PROFILER.scope("gdn.chunked"):
                core = gdn.chunked(mixed, 0, self.kd, 2 * self.kd, g, beta, self.states[slot, idx], self.hv_lin, self.hk_lin)
        else:                  # one token per sequence
            mixed = basic.conv_silu_step(proj[:, :cw], lw.conv_w, self.tails[:, idx], slots_t)
            core = gdn.step(self.states[:, idx], slots_t, mixed, 0, self.kd, 2 * self.kd, g, beta, self.hv_lin, self.hk_lin)
        z = proj[:, cw:].unflatten(1, (self.hv_lin, 128))
        y = basic.gated_rmsnorm(core, z, lw.gdn_norm, cfg.rms_norm_eps)
        with PROFILER.scope("lin.out+ar.attn"):
            return self._row_parallel(y.view(t, self.vd), lw.out)

    def _attend(self, idx: int, lw: LayerWeights, proj: torch.Tensor, t: int, positions, kv_slots, meta, eps) -> torch.Tensor:
        """QK-norm + RoPE + cache append + attention of one full-attention layer, for either cache dtype."""
        cfg = self.cfg
        gate_mul = 2 if cfg.attn_output_gate else 1
        qw = self.hq * 128 * gate_mul
        win, sinks = self.attention_window, self.attention_sinks

        def rope_append(slots, kc, vc):
            return attention.qk_norm_rope_append(
                proj, 0, 128 * gate_mul, cfg.attn_output_gate, proj, qw, proj, qw + self.hkv * 128, lw.q_norm, lw.k_norm,
                True, eps, self.inv_freq, cfg.rotary_dim, positions, slots, kc, vc, self.hq, self.hkv)

        if self.kv8 is None:
            kc, vc = self.k_cache[idx], self.v_cache[idx]
            q, gate = rope_append(kv_slots, kc, vc)
            if meta["mode"] == "prefill":
                with PROFILER.scope("full.attn_kernel"):
                    return attention.prefill(q, kc, vc, meta["block_table"], meta["q_start"], meta["q_len"], meta["kv_len"],
                                             meta["max_q_len"], gate=gate, window=win, sinks=sinks)
            return attention.decode(q, kc, vc, meta["block_table"], meta["kv_len"], gate=gate, max_kv_len=meta["max_kv_len"],
                                    window=win, sinks=sinks)
        c = self.kv8
        k8, v8, ks, vs, vm = c.layer(idx)
        if meta["mode"] == "prefill":
            # past rows come back dequantised, the chunk's own rows stay exact bf16; a row's position is its staging slot
            attention.kv8_dequantize(c.fmt, k8, v8, ks, vs, meta["block_table"][0], meta["past"], self.stage_k, self.stage_v, vm)
            q, gate = rope_append(positions, self.stage_k, self.stage_v)
            attention.kv8_quantize(c.fmt, self.stage_k, self.stage_v, positions, kv_slots, k8, v8, ks, vs, vm)
            with PROFILER.scope("full.attn_kernel"):
                return attention.prefill(q, self.stage_k, self.stage_v, self._ident_bt, meta["q_start"], meta["q_len"],
                                         meta["kv_len"], meta["max_q_len"], gate=gate, window=win, sinks=sinks)
        rows = self._rows[:t]
        q, gate = rope_append(rows, self.dstage_k, self.dstage_v)
        attention.kv8_quantize(c.fmt, self.dstage_k, self.dstage_v, rows, kv_slots, k8, v8, ks, vs, vm)
        return attention.decode_kv8(c.fmt, q, k8, v8, ks, vs, meta["block_table"], meta["kv_len"], gate=gate,
                                    max_kv_len=meta["max_kv_len"], window=win, sinks=sinks, v_min=vm)

    def _full_attn(self, li: int, lw: LayerWeights, x: torch.Tensor, t: int, positions, kv_slots, meta) -> torch.Tensor:
        idx = self.full_layers.index(li)
        proj = self._col_parallel(x, lw.proj)
        o = self._attend(idx, lw, proj, t, positions, kv_slots, meta, self.cfg.rms_norm_eps)
        return self._row_parallel(o.view(t, self.hq * 128), lw.out)

    def _embed(self, ids: torch.Tensor) -> torch.Tensor:
        h = basic.embedding(ids, self.w.embed, self.w.vocab_lo, self.w.vocab_hi)
        return h if self.w.embed_replicated else self.comm.all_reduce(h)

    def _forward(self, ids, positions, kv_slots, meta, slot, slots_t, logits_rows: torch.Tensor | None):
        cfg, w = self.cfg, self.w
        t = ids.numel()
        h = self._embed(ids)
        delta = None
        for i, lw in enumerate(w.layers):
            if delta is None:
                x = basic.rmsnorm(h, lw.in_ln, cfg.rms_norm_eps, True)
            else:
                x = basic.add_rmsnorm(h, delta, lw.in_ln, cfg.rms_norm_eps, True)
            if lw.kind == "linear":
                d_attn = self._linear_attn(i, lw, x, t, slots_t, slot)
            else:
                d_attn = self._full_attn(i, lw, x, t, positions, kv_slots, meta)
            delta = self._mlp(lw, h, d_attn)
        if logits_rows is not None and self.keep_hidden:
            self.hidden_rows = basic.add_rmsnorm(h, delta, w.final_norm, cfg.rms_norm_eps, True)
            x = self.hidden_rows.index_select(0, logits_rows)
        elif logits_rows is not None:
            basic.add_(h, delta)
            hs = h.index_select(0, logits_rows)
            x = basic.rmsnorm(hs, w.final_norm, cfg.rms_norm_eps, True)
        else:
            x = basic.add_rmsnorm(h, delta, w.final_norm, cfg.rms_norm_eps, True)
        logits = gemm.linear(x, w.lm_head, out_f32=True)
        return logits

    def _forward_sp(self, ids, positions, kv_slots, meta, slot, logits_rows: torch.Tensor, rows: int) -> torch.Tensor:
        """One prefill chunk with the residual stream sharded by token rows over the tensor-parallel ranks.

        Rank r keeps rows [r*rows, (r+1)*rows) of the hidden state.  Each sub-layer is: reduce (partials of the
        previous row-parallel GEMM) + residual add + RMSNorm on the own rows, gathered into every rank's activation
        buffer -> column-parallel GEMM that consumes the buffer tile by tile as the rows arrive -> token mixer /
        activation on this rank's heads or features -> row-parallel GEMM that pushes its partial tiles to the row
        owners.  The same math, with the same roundings, as ``_forward``; norms and residual adds run on T / world
        rows and no stand-alone collective is on the path (the reference all-reduces after every row-parallel
        projection and norms the replicated tensor, cpp_engine/engine/qwen_engine.cpp:1942-2037, 3236-3245)."""
        cfg, w, comm = self.cfg, self.w, self.comm
        t = ids.numel()
        eps = cfg.rms_norm_eps
        own = slice(comm.rank * rows, (comm.rank + 1) * rows)
        h = self._embed(ids[own]) if w.embed_replicated else self._embed(ids)[own].clone()
        self._sp = True
        try:
            first = True
            for i, lw in enumerate(w.layers):
                x = comm.reduce_norm_gather(h, lw.in_ln, eps, True, with_partials=not first)
                first = False
                if lw.kind == "linear":
                    self._linear_attn(i, lw, x, t, None, slot)
                else:
                    self._full_attn(i, lw, x, t, positions, kv_slots, meta)
                self._mlp(lw, h, None)
            x = comm.reduce_norm_gather(h, w.final_norm, eps, True)
            comm.wait_gather(rows)
            if self.keep_hidden:
                self.hidden_rows = x.clone()       # the gathered buffer is overwritten by the next chunk
        finally:
            self._sp = False
        return gemm.linear(x.index_select(0, logits_rows), w.lm_head, out_f32=True)

    def _forward_decode(self, ids, positions, kv_slots, meta, slots_t) -> torch.Tensor:
        """Decode step for up to 32 sequences: FP8 projections through the weight-streaming kernel (activations
        handed over as E4M3 terms by the fused norm / activation kernels), one fused launch for the whole
        Gated-DeltaNet token mixer.  Same math as ``_forward``; 9 launches per linear layer instead of 16."""
        cfg, w = self.cfg, self.w
        t = ids.numel()
        _, terms = gemm.stream_layout(t)
        eps = cfg.rms_norm_eps
        h = self._embed(ids)
        delta = None
        for i, lw in enumerate(w.layers):
            x, xs = basic.rmsnorm_split(h, delta, lw.in_ln, terms, eps, True, want_bf16=lw.kind == "linear")
            proj = gemm.linear_stream(None, lw.proj, xsplit=xs)
            if lw.kind == "linear":
                idx = self.lin_layers.index(i)
                y = gdn.decode_fused(proj, x, lw.ab.weight, lw.a_log, lw.dt_bias, lw.conv_w, self.tails[:, idx],
                                     self.states[:, idx], slots_t, lw.gdn_norm, self.hv_lin, self.hk_lin, eps)
                d_attn = self._stream_row_parallel(y, lw.out)
            else:
                o = self._attend(self.full_layers.index(i), lw, proj, t, positions, kv_slots, meta, eps)
                d_attn = self._stream_row_parallel(o.view(t, self.hq * 128), lw.out)
            _, xs2 = basic.rmsnorm_split(h, d_attn, lw.post_ln, terms, eps, True, want_bf16=False)
            gu = gemm.linear_stream(None, lw.gate_up, xsplit=xs2)
            delta = self._stream_row_parallel(None, lw.down, basic.silu_mul_split(gu, terms))
        x = basic.add_rmsnorm(h, delta, w.final_norm, eps, True)
        return gemm.linear(x, w.lm_head, out_f32=True)

    def _next_tokens(self, logits: torch.Tensor, sampling=None, u: torch.Tensor | None = None,
                     counts: torch.Tensor | None = None) -> torch.Tensor:
        """Greedy arg-max over the vocabulary shards, or (``sampling``: ops.sampling.DeviceSampling, ``u``: fp32 [B]
        uniforms) a temperature / top-k / top-p / min-p draw on the device."""
        if sampling is None:
            idx, val = basic.argmax(logits, self.w.head_lo, True)
            return self.comm.argmax_merge(idx, val)
        from ..ops import sampling as smp
        return smp.sample(logits.float(), sampling, u.to(self.device, torch.float32), self.w.head_lo, self.comm, counts)

    # ---- public: prefill one sequence (chunked), returns the next token id tensor [1] (device)
    @torch.no_grad()
    def prefill(self, slot: int, token_ids: torch.Tensor, chunk: int = 8192, host_tokens: list[int] | None = None,
                sampling=None, u: torch.Tensor | None = None, counts: torch.Tensor | None = None) -> torch.Tensor:
        """token_ids: int32 device tensor [T]. Appends to the slot's context. Returns greedy next token.
        With the prefix cache enabled a fresh slot first resumes from the longest cached prefix of the prompt and
        chunks are cut at the snapshot points (``host_tokens`` saves the device-to-host copy of the ids)."""
        st = self.seqs[slot]
        l0 = _lib.LAUNCHES
        nxt = None
        total = token_ids.numel()
        cuts, s = [], 0
        if self.prefix_cache is not None and st.length == 0:
            # fresh slot: positions equal indices into token_ids
            host_tokens = host_tokens if host_tokens is not None else token_ids.tolist()
            self._restore_prefix(st, host_tokens)
            s = st.length
            cuts = self.prefix_cache.boundaries(st.length, total)
        while s < total:
            e = min(total, s + chunk)
            nxt_cut = next((c for c in cuts if c > s), None)
            if nxt_cut is not None and nxt_cut < e:
                e = nxt_cut
            ids = token_ids[s:e]
            t = ids.numel()
            self._ensure_blocks(st, st.length + t)
            pos = torch.arange(st.length, st.length + t, dtype=torch.int32, device=self.device)
            bt_row = self.block_table[slot]
            kv_slots = (bt_row[(pos // self.block_size).long()] * self.block_size + pos % self.block_size).to(torch.int32)
            i32 = lambda v: torch.tensor([v], dtype=torch.int32, device=self.device)
            meta = {"mode": "prefill", "block_table": self.block_table[slot:slot + 1], "q_start": i32(0),
                    "q_len": i32(t), "kv_len": i32(st.length + t), "max_q_len": t, "past": st.length}
            rows = torch.tensor([t - 1], dtype=torch.int64, device=self.device)
            sp_rows = self.comm.sp_rows(t, self.cfg.hidden_size) if hasattr(self.comm, "sp_rows") else 0
            if sp_rows:
                logits = self._forward_sp(ids, pos, kv_slots, meta, slot, rows, sp_rows)
            else:
                logits = self._forward(ids, pos, kv_slots, meta, slot, None, rows)
            self.last_logits = logits                  # last row of the latest chunk (fp32 [1, vocab])
            st.length += t
            self.prefill_tokens_computed += t
            if e in cuts:
                self._snapshot_prefix(st, host_tokens)
            if e >= total:
                nxt = self._next_tokens(logits, sampling, u, counts)
            s = e
        self.launches = _lib.LAUNCHES - l0
        return nxt

    # ---- public: one decode step for a batch of slots
    def _decode_buffers(self, b: int):
        dev = self.device
        return {
            "ids": torch.zeros(b, dtype=torch.int32, device=dev),
            "pos": torch.zeros(b, dtype=torch.int32, device=dev),
            "kv_slots": torch.zeros(b, dtype=torch.int32, device=dev),
            "slots": torch.zeros(b, dtype=torch.int32, device=dev),
            "kv_len": torch.ones(b, dtype=torch.int32, device=dev),
            "bt": torch.zeros(b, self.max_blocks_per_seq, dtype=torch.int32, device=dev),
        }

    def _decode_body(self, buf, max_kv_len: int) -> torch.Tensor:
        meta = {"mode": "decode", "block_table": buf["bt"], "kv_len": buf["kv_len"], "max_kv_len": max_kv_len}
        if buf["ids"].numel() <= gemm.STREAM_MAX_T and self.fused_decode:
            logits = self._forward_decode(buf["ids"], buf["pos"], buf["kv_slots"], meta, buf["slots"])
        else:
            logits = self._forward(buf["ids"], buf["pos"], buf["kv_slots"], meta, None, buf["slots"], None)
        buf["logits"] = logits          # kept for device-side sampling after the (possibly replayed) step
        return self._next_tokens(logits)

    @torch.no_grad()
    def decode(self, slots: list[int], token_ids: torch.Tensor, use_graph: bool = True, sampling=None,
               u: torch.Tensor | None = None, counts: torch.Tensor | None = None) -> torch.Tensor:
        """One new token for each slot. token_ids: int32 device tensor [B]. Returns next tokens [B] (device): greedy,
        or drawn on the device from the step's logits when ``sampling`` / ``u`` are given (see ``_next_tokens``)."""
        b = len(slots)
        sts = [self.seqs[s] for s in slots]
        for st in sts:
            self._ensure_blocks(st, st.length + 1)
        max_len = max(st.length for st in sts) + 1
        bucket = 1 << max(10, (max_len - 1).bit_length())  # context bucket fixes the decode-attention split count
        key = (b, bucket)
        entry = self._graphs.get(key)
        if entry is None:
            entry = {"buf": self._decode_buffers(b), "graph": None, "out": None}
            self._graphs[key] = entry
        buf = entry["buf"]
        host = torch.tensor([[st.length, st.length + 1, st.slot,
                              st.blocks[st.length // self.block_size] * self.block_size + st.length % self.block_size]
                             for st in sts], dtype=torch.int32)
        dev = host.to(self.device, non_blocking=True)
        buf["ids"].copy_(token_ids)
        buf["pos"].copy_(dev[:, 0])
        buf["kv_len"].copy_(dev[:, 1])
        buf["slots"].copy_(dev[:, 2])
        buf["kv_slots"].copy_(dev[:, 3])
        buf["bt"].copy_(self.block_table[buf["slots"].long()])
        if not use_graph:
            l0 = _lib.LAUNCHES
            out = self._decode_body(buf, bucket)
            self.launches = _lib.LAUNCHES - l0
        else:
            if entry["graph"] is None:
                # warm-up outside capture (lazy kernel attribute set-up, workspaces), on state copies
                saved = (self.states.clone(), self.tails.clone())
                self._decode_body(buf, bucket)
                torch.cuda.synchronize()
                self.states.copy_(saved[0])
                self.tails.copy_(saved[1])
                del saved
                gph = torch.cuda.CUDAGraph()
                l0 = _lib.LAUNCHES
                with torch.cuda.graph(gph):
                    entry["out"] = self._decode_body(buf, bucket)
                entry["graph"] = gph
                entry["launches"] = _lib.LAUNCHES - l0
                # capture does not execute: run the step now
            entry["graph"].replay()
            self.launches = entry["launches"]
            out = entry["out"]
        for st in sts:
            st.length += 1
        self.last_logits = buf["logits"]               # [B, vocab shard] fp32 of this step (log-probabilities, sampling)
        if sampling is not None:
            out = self._next_tokens(buf["logits"], sampling, u, counts)
        return out

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new_tokens: int, chunk: int = 8192, eos: int | None = None) -> list[int]:
        slot = self.allocate()
        try:
            tok = self.prefill(slot, prompt.to(self.device, torch.int32), chunk)
            out = [int(tok.item())]
            while len(out) < max_new_tokens and (eos is None or out[-1] != eos):
                tok = self.decode([slot], tok.to(torch.int32))
                out.append(int(tok.item()))
            return out
        finally:
            self.free(slot)


def build_synthetic(cfg: QwenHybridConfig, device="cuda", seed: int = 0, tp_rank: int = 0, tp_world: int = 1,
                    **rt_kwargs) -> QwenHybridRuntime:
    """Random-init model of the given shape, generated on the device with the checkpoint writer's generator."""
    w = QwenHybridWeights(cfg, synth_state(cfg, seed, device), device, tp_rank, tp_world)
    return QwenHybridRuntime(cfg, w, **rt_kwargs)
