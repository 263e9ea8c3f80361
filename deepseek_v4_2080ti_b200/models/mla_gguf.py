"""GGUF checkpoints of the MLA + sparse-indexer MoE family (GLM-style ``glm-dsa`` naming): metadata <-> config, the
tensor-name map, a writer for synthetic checkpoints, and the reader that hands the GPU weight loader *raw* quantised
blocks (``RawQuant``) so that nothing is dequantised or re-quantised on the way to the in-register-decode GEMMs.

Naming follows the reference's source-name table (src/loader/mappings/glm_dsa.py:7-63): ``token_embd`` / ``output`` /
``output_norm``; per layer ``attn_q_a`` (+ ``_norm``), ``attn_q_b``, ``attn_kv_a_mqa`` (+ ``attn_kv_a_norm``),
``attn_k_b`` [heads, kv_lora, nope] and ``attn_v_b`` [heads, v, kv_lora] (the absorbed halves of the kv up-projection),
``attn_output``, ``indexer.{attn_q_b, attn_k, k_norm, proj}``, dense ``ffn_{gate,up,down}`` or MoE ``ffn_gate_inp``,
``exp_probs_b.bias``, ``ffn_{gate,up,down}_exps`` [experts, rows, cols], ``ffn_{gate,up,down}_shexp``; multi-token
prediction blocks sit after the last layer with ``nextn.{eh_proj, enorm, hnorm}`` (:57-63).
"""
from __future__ import annotations

from typing import Any, Iterator

import torch

from ..formats import gguf as G
from ..formats.gguf import BLOCK_BYTES, BLOCK_ELEMS, GGMLType
from .mla_moe import MlaMoeConfig

ARCH = "glm-dsa"
DEFAULT_MIX = {"attn": "Q8_0", "ffn": "Q4_K", "gate_up": "Q2_K", "down": "IQ3_XXS"}
_SCORE = {"softmax": 1, "sigmoid": 2, "sqrtsoftplus": 3}
_SCORE_INV = {v: k for k, v in _SCORE.items()}


# ---------------------------------------------------------------------------------------------- raw blocks
class RawQuant:
    """Rows of raw GGUF blocks: ``raw`` uint8 [n, k / block_elems * block_bytes] standing for a logical [n, k] matrix."""
    __slots__ = ("raw", "t", "n", "k")

    def __init__(self, raw: torch.Tensor, t: GGMLType, n: int, k: int):
        self.t = GGMLType(t)
        self.n, self.k = int(n), int(k)
        self.raw = raw.reshape(self.n, -1)
        assert self.raw.shape[1] == self.k // BLOCK_ELEMS[self.t] * BLOCK_BYTES[self.t], (self.raw.shape, self.t, n, k)

    @property
    def shape(self) -> tuple[int, int]:
        return (self.n, self.k)

    def to(self, device) -> "RawQuant":
        return RawQuant(self.raw.to(device), self.t, self.n, self.k)

    def rows(self, lo: int, hi: int) -> "RawQuant":
        return RawQuant(self.raw[lo:hi], self.t, hi - lo, self.k)

    def cols(self, lo: int, hi: int) -> "RawQuant | None":
        """Input-dimension slice on block boundaries (None when the cut would split a block)."""
        be, bb = BLOCK_ELEMS[self.t], BLOCK_BYTES[self.t]
        if lo % be or hi % be:
            return None
        return RawQuant(self.raw.reshape(self.n, self.k // be, bb)[:, lo // be:hi // be].reshape(self.n, -1).contiguous(),
                        self.t, self.n, hi - lo)

    def dequant(self) -> torch.Tensor:
        return G.dequantize(self.raw.contiguous(), self.t, self.k)

    @staticmethod
    def cat(parts: list["RawQuant"]) -> "RawQuant | None":
        """Row-wise concatenation (None unless every part has the same type and width)."""
        if any(p.t != parts[0].t or p.k != parts[0].k for p in parts):
            return None
        return RawQuant(torch.cat([p.raw for p in parts]), parts[0].t, sum(p.n for p in parts), parts[0].k)


# ---------------------------------------------------------------------------------------------- metadata
def metadata(cfg: MlaMoeConfig, context_length: int = 8192) -> dict[str, Any]:
    a = ARCH
    return {"general.architecture": a, "general.name": "synthetic-glm-dsa",
            f"{a}.block_count": cfg.num_layers + cfg.mtp_layers, f"{a}.nextn_predict_layers": cfg.mtp_layers,
            f"{a}.context_length": context_length, f"{a}.embedding_length": cfg.hidden_size, f"{a}.vocab_size": cfg.vocab_size,
            f"{a}.feed_forward_length": cfg.dense_intermediate, f"{a}.leading_dense_block_count": cfg.first_dense_layers,
            f"{a}.attention.head_count": cfg.num_heads, f"{a}.attention.head_count_kv": 1,
            f"{a}.attention.q_lora_rank": cfg.q_lora_rank, f"{a}.attention.kv_lora_rank": cfg.kv_lora_rank,
            f"{a}.attention.key_length": cfg.qk_head_dim, f"{a}.attention.value_length": cfg.v_head_dim,
            f"{a}.rope.dimension_count": cfg.qk_rope_dim, f"{a}.rope.freq_base": float(cfg.rope_theta),
            f"{a}.attention.layer_norm_rms_epsilon": float(cfg.rms_norm_eps),
            f"{a}.attention.indexer.head_count": cfg.index_heads, f"{a}.attention.indexer.key_length": cfg.index_dim,
            f"{a}.attention.indexer.top_k": cfg.index_topk,
            f"{a}.expert_count": cfg.num_experts, f"{a}.expert_used_count": cfg.experts_per_token,
            f"{a}.expert_shared_count": cfg.num_shared_experts, f"{a}.expert_feed_forward_length": cfg.expert_intermediate,
            f"{a}.expert_gating_func": _SCORE[cfg.score_func], f"{a}.expert_weights_scale": float(cfg.route_scale),
            f"{a}.expert_weights_norm": bool(cfg.norm_topk)}


def config_from_metadata(md: dict[str, Any], tensors: dict | None = None) -> MlaMoeConfig:
    a = str(md.get("general.architecture", ARCH))
    g = lambda k, d=0: md.get(f"{a}.{k}", d)
    mtp = int(g("nextn_predict_layers", 0))
    key_len, rope = int(g("attention.key_length")), int(g("rope.dimension_count"))
    return MlaMoeConfig(
        vocab_size=int(g("vocab_size")), hidden_size=int(g("embedding_length")), num_layers=int(g("block_count")) - mtp,
        first_dense_layers=int(g("leading_dense_block_count", 0)), dense_intermediate=int(g("feed_forward_length", 0)),
        q_lora_rank=int(g("attention.q_lora_rank", 0)), kv_lora_rank=int(g("attention.kv_lora_rank")),
        num_heads=int(g("attention.head_count")), qk_nope_dim=key_len - rope, qk_rope_dim=rope,
        v_head_dim=int(g("attention.value_length")), rope_theta=float(g("rope.freq_base", 1e4)),
        rms_norm_eps=float(round(float(g("attention.layer_norm_rms_epsilon", 1e-6)), 12)),
        index_heads=int(g("attention.indexer.head_count", 0)), index_dim=int(g("attention.indexer.key_length", 0)),
        index_topk=int(g("attention.indexer.top_k", 0)), num_experts=int(g("expert_count")),
        experts_per_token=int(g("expert_used_count")), num_shared_experts=int(g("expert_shared_count", 0)),
        expert_intermediate=int(g("expert_feed_forward_length")), score_func=_SCORE_INV[int(g("expert_gating_func", 2))],
        route_scale=float(g("expert_weights_scale", 1.0)), norm_topk=bool(g("expert_weights_norm", True)),
        expert_format="bf16", mtp_layers=mtp)


# ---------------------------------------------------------------------------------------------- name map
GLOBAL = {"token_embd.weight": "embed.weight", "output_norm.weight": "norm.weight", "output.weight": "head.weight"}
ATTN = {"attn_norm.weight": "attn_norm.weight", "ffn_norm.weight": "ffn_norm.weight", "attn_q_a.weight": "attn.wq_a.weight",
        "attn_q_a_norm.weight": "attn.q_norm.weight", "attn_q_b.weight": "attn.wq_b.weight", "attn_q.weight": "attn.wq.weight",
        "attn_kv_a_mqa.weight": "attn.wkv_a.weight", "attn_kv_a_norm.weight": "attn.kv_norm.weight",
        "attn_output.weight": "attn.wo.weight", "indexer.attn_q_b.weight": "attn.indexer.wq_b.weight",
        "indexer.attn_k.weight": "attn.indexer.wk.weight", "indexer.k_norm.weight": "attn.indexer.k_norm.weight",
        "indexer.proj.weight": "attn.indexer.weights_proj.weight"}
DENSE = {"ffn_gate.weight": "ffn.w1.weight", "ffn_up.weight": "ffn.w3.weight", "ffn_down.weight": "ffn.w2.weight"}
MOE = {"ffn_gate_inp.weight": "ffn.gate.weight", "exp_probs_b.bias": "ffn.gate.bias",
       "ffn_gate_shexp.weight": "ffn.shared_experts.w1.weight", "ffn_up_shexp.weight": "ffn.shared_experts.w3.weight",
       "ffn_down_shexp.weight": "ffn.shared_experts.w2.weight"}
EXPERTS = {"ffn_gate_exps.weight": "w1", "ffn_up_exps.weight": "w3", "ffn_down_exps.weight": "w2"}
NEXTN = {"nextn.enorm.weight": "enorm.weight", "nextn.hnorm.weight": "hnorm.weight"}
OPTIONAL = ("indexer.k_norm.bias", "nextn.shared_head_norm.weight")     # read by the reference, unused by this runtime


def layer_suffixes(cfg: MlaMoeConfig, layer: int) -> tuple[str, ...]:
    """GGUF tensor suffixes (after ``blk.N.``) layer ``layer`` must have; layers past ``num_layers`` are MTP blocks."""
    out = ["attn_norm.weight", "ffn_norm.weight", "attn_kv_a_mqa.weight", "attn_kv_a_norm.weight", "attn_k_b.weight",
           "attn_v_b.weight", "attn_output.weight"]
    out += ["attn_q_a.weight", "attn_q_a_norm.weight", "attn_q_b.weight"] if cfg.q_lora_rank > 0 else ["attn_q.weight"]
    if cfg.index_heads > 0:
        out += ["indexer.attn_q_b.weight", "indexer.attn_k.weight", "indexer.k_norm.weight", "indexer.proj.weight"]
    if layer < cfg.first_dense_layers:
        out += list(DENSE)
    else:
        out += ["ffn_gate_inp.weight", "exp_probs_b.bias", *EXPERTS]
        if cfg.num_shared_experts:
            out += ["ffn_gate_shexp.weight", "ffn_up_shexp.weight", "ffn_down_shexp.weight"]
    if layer >= cfg.num_layers:
        out += ["nextn.eh_proj.weight", *NEXTN]
    return tuple(out)


# ---------------------------------------------------------------------------------------------- writer
def _pick(tname: str, k: int) -> GGMLType:
    """The requested type when the row length holds whole blocks, else Q8_0, else F32."""
    t = GGMLType[tname]
    if k % BLOCK_ELEMS[t] == 0:
        return t
    return GGMLType.Q8_0 if k % 32 == 0 else GGMLType.F32


def _enc(w: torch.Tensor, t: GGMLType) -> torch.Tensor:
    if t == GGMLType.F32:
        return w.float().contiguous().view(torch.uint8)
    return G.quantize(w.float().reshape(-1, w.shape[-1]), t)


def state_to_gguf(cfg: MlaMoeConfig, state: Iterator[tuple[str, torch.Tensor]], mix: dict[str, str] | None = None
                  ) -> Iterator[tuple[str, torch.Tensor, GGMLType, tuple[int, ...]]]:
    """(gguf name, raw bytes, type, logical shape) for every tensor of a state in this package's key naming (bf16
    experts).  Experts are stacked per layer; identical expert tensors (a benchmark's small pool) are quantised once."""
    mix = dict(DEFAULT_MIX, **(mix or {}))
    inv = {v: k for k, v in {**ATTN, **DENSE, **MOE}.items()}
    kinds = {"attn_q_a": "attn", "attn_q_b": "attn", "attn_q": "attn", "attn_kv_a_mqa": "attn", "attn_output": "attn",
             "indexer": "attn"}
    pending: dict[tuple[str, str], dict[int, torch.Tensor]] = {}
    eh: dict[str, dict[str, torch.Tensor]] = {}
    n, v_, c = cfg.qk_nope_dim, cfg.v_head_dim, cfg.kv_lora_rank

    def blk(key: str) -> tuple[str, str]:
        if key.startswith("layers."):
            _, li, rest = key.split(".", 2)
            return f"blk.{int(li)}.", rest
        _, j, rest = key.split(".", 2)
        return f"blk.{cfg.num_layers + int(j)}.", rest

    for key, w in state:
        if key == "embed.weight" or key == "head.weight":
            name = "token_embd.weight" if key == "embed.weight" else "output.weight"
            t = _pick(mix["ffn"], w.shape[1])
            yield name, _enc(w, t), t, tuple(w.shape)
            continue
        if key == "norm.weight":
            yield "output_norm.weight", _enc(w, GGMLType.F32), GGMLType.F32, tuple(w.shape)
            continue
        p, rest = blk(key)
        if rest == "attn.wkv_b.weight":
            wb = w.float().view(cfg.num_heads, n + v_, c)
            kb = wb[:, :n].transpose(1, 2).contiguous()                   # [H, C, N]
            vb = wb[:, n:].contiguous()                                    # [H, V, C]
            for name, m in (("attn_k_b.weight", kb), ("attn_v_b.weight", vb)):
                t = _pick(mix["attn"], m.shape[-1])
                yield p + name, _enc(m, t), t, tuple(m.shape)
            continue
        if ".experts." in rest:
            e, wn = rest.split(".experts.")[1].split(".")[:2]
            if rest.endswith(".scale"):
                raise ValueError("FP4 expert states are not exported; build the state with expert_format='bf16'")
            d = pending.setdefault((p, wn), {})
            d[int(e)] = w
            if len(d) == cfg.num_experts:
                gname = {v: k for k, v in EXPERTS.items()}[wn]
                t = _pick(mix["down" if wn == "w2" else "gate_up"], w.shape[1])
                cache: dict[int, torch.Tensor] = {}
                raws = []
                for i in range(cfg.num_experts):
                    key_id = d[i].data_ptr()
                    if key_id not in cache:
                        cache[key_id] = _enc(d[i], t)
                    raws.append(cache[key_id])
                yield p + gname, torch.stack(raws), t, (cfg.num_experts, *w.shape)
                del pending[(p, wn)]
            continue
        if rest in ("e_proj.weight", "h_proj.weight"):
            d2 = eh.setdefault(p, {})
            d2[rest] = w
            if len(d2) == 2:
                m = torch.cat([d2["e_proj.weight"].float(), d2["h_proj.weight"].float()], 1)
                t = _pick(mix["ffn"], m.shape[1] // 2)
                yield p + "nextn.eh_proj.weight", _enc(m, t), t, tuple(m.shape)
            continue
        if rest in ("enorm.weight", "hnorm.weight"):
            yield p + "nextn." + rest, _enc(w, GGMLType.F32), GGMLType.F32, tuple(w.shape)
            continue
        name = inv[rest]
        if w.ndim == 1 or name == "ffn_gate_inp.weight":
            yield p + name, _enc(w, GGMLType.F32), GGMLType.F32, tuple(w.shape)
            continue
        kind = next((k for pre, k in kinds.items() if name.startswith(pre)), "ffn")
        t = _pick(mix[kind], w.shape[1])
        yield p + name, _enc(w, t), t, tuple(w.shape)
    assert not pending, f"incomplete expert stacks: {sorted(pending)[:3]}"


def write_synthetic_gguf(path: str, cfg: MlaMoeConfig, mix: dict[str, str] | None = None, seed: int = 0, std: float = 0.02,
                         device="cpu", expert_pool: int | None = None) -> None:
    from dataclasses import replace
    from . import mla_moe
    src = replace(cfg, expert_format="bf16")
    G.write_gguf(path, metadata(cfg), ((n, r.cpu(), t, s) for n, r, t, s in
                                       state_to_gguf(src, mla_moe.synth_state(src, seed, device, std, expert_pool=expert_pool), mix)))


# ---------------------------------------------------------------------------------------------- reader
def read_state(store, cfg: MlaMoeConfig, device=None, expert_range: tuple[int, int] | None = None,
               layer_range: tuple[int, int] | None = None) -> Iterator[tuple[str, Any]]:
    """State entries in this package's key naming from a GGUF tensor store (``models.gqa_moe.TensorStore``): plain
    tensors for norms, biases, the router, the embedding table (dequantised to bf16) and the kv up-projection
    (rebuilt from its absorbed halves); ``RawQuant`` for every quantised matrix.  ``expert_range`` / ``layer_range``
    skip what a rank does not hold before anything is copied to ``device``."""
    n, v_, c = cfg.qk_nope_dim, cfg.v_head_dim, cfg.kv_lora_rank
    mv = (lambda x: x.to(device)) if device is not None else (lambda x: x)

    def plain(name: str) -> torch.Tensor:
        raw, t, shape = store.get(name)
        if t == GGMLType.F32:
            return mv(store.f32(name))
        return G.dequantize(mv(raw.reshape(-1, raw.shape[-1]).contiguous()), t, shape[-1]).reshape(shape)

    def mat(name: str):
        raw, t, shape = store.get(name)
        if t == GGMLType.F32:
            return mv(store.f32(name)).to(torch.bfloat16)
        return RawQuant(mv(raw.reshape(shape[-2], -1).contiguous()), t, shape[-2], shape[-1])

    names = set(store.names())
    if layer_range is None or layer_range[0] == 0 or cfg.mtp_layers:
        yield "embed.weight", plain("token_embd.weight").to(torch.bfloat16)
    yield "norm.weight", plain("output_norm.weight")
    yield "head.weight", mat("output.weight" if "output.weight" in names else "token_embd.weight")
    for li in range(cfg.num_layers + cfg.mtp_layers):
        is_mtp = li >= cfg.num_layers
        if not is_mtp and layer_range is not None and not (layer_range[0] <= li < layer_range[1]):
            continue
        p = f"blk.{li}."
        sp = f"mtp.{li - cfg.num_layers}." if is_mtp else f"layers.{li}."
        for suffix in layer_suffixes(cfg, li):
            name = p + suffix
            if suffix in ATTN or suffix in DENSE or suffix in MOE:
                key = sp + {**ATTN, **DENSE, **MOE}[suffix]
                yield key, (plain(name) if suffix.endswith(("norm.weight", ".bias")) or suffix == "ffn_gate_inp.weight"
                            else mat(name))
            elif suffix == "attn_k_b.weight":
                kb = plain(name).float().reshape(cfg.num_heads, c, n)
                vb = plain(p + "attn_v_b.weight").float().reshape(cfg.num_heads, v_, c)
                yield sp + "attn.wkv_b.weight", torch.cat([kb.transpose(1, 2), vb], 1).reshape(-1, c).to(torch.bfloat16)
            elif suffix == "attn_v_b.weight":
                continue
            elif suffix in EXPERTS:
                raw, t, shape = store.get(name)
                lo, hi = expert_range or (0, cfg.num_experts)
                for e in range(lo, hi):
                    key = sp + f"ffn.experts.{e}.{EXPERTS[suffix]}.weight"
                    if t == GGMLType.F32:
                        yield key, mv(raw[e].contiguous().view(torch.float32).reshape(shape[1:])).to(torch.bfloat16)
                    else:
                        yield key, RawQuant(mv(raw[e].reshape(shape[1], -1).contiguous()), t, shape[1], shape[2])
            elif suffix == "nextn.eh_proj.weight":
                m = mat(name)
                h = cfg.hidden_size
                if isinstance(m, RawQuant):
                    parts = (m.cols(0, h), m.cols(h, 2 * h))
                    if parts[0] is None:
                        d = m.dequant().to(torch.bfloat16)
                        parts = (d[:, :h].contiguous(), d[:, h:].contiguous())
                else:
                    parts = (m[:, :h].contiguous(), m[:, h:].contiguous())
                yield sp + "e_proj.weight", parts[0]
                yield sp + "h_proj.weight", parts[1]
            elif suffix in NEXTN:
                yield sp + NEXTN[suffix], plain(name)
