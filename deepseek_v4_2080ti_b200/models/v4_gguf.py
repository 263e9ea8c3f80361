"""GGUF checkpoints of the DeepSeek-V4 architecture (``general.architecture = deepseek4``): metadata <-> ``V4Config``,
the tensor-name table, a validator that reports every mismatch at once, a writer for synthetic checkpoints and the
loader that fills the weight dictionary of the fp32 block runtime (``models/v4_block_ref.py``).

The table below is the whole mapping: one row per kind of tensor, ``{L}`` standing for the layer number.  GGUF names
follow the reference's source-name list (src/loader/mappings/deepseek_v4.py:62-135): ``token_embd`` / ``output`` /
``output_norm`` / ``output_hc_{fn,base,scale}``; per block ``attn_sinks``, ``attn_q_a`` (+ ``_norm``), ``attn_q_b``,
``attn_kv`` (+ ``attn_kv_a_norm``), ``attn_output_{a,b}``, ``attn_norm``, ``ffn_gate_inp``, ``ffn_gate_tid2eid`` (hash
layers) or ``exp_probs_b.bias``, ``ffn_{gate,down,up}_exps`` stacked over experts, ``ffn_{gate,down,up}_shexp``,
``ffn_norm``, ``hc_{attn,ffn}_{fn,base,scale}``, ``attn_compressor_{ape,kv,gate,norm}`` on compressed layers and
``indexer.{attn_q_b,proj}`` + ``indexer_compressor_{ape,kv,gate,norm}`` on indexer layers.  Matrices are stored
``[out, in]`` in this package's reader convention (GGUF lists the dimensions innermost first), so no tensor is
transposed on the way in; stacked expert tensors are ``[experts, out, in]`` and split per expert.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

from ..formats import gguf as G
from ..formats.gguf import BLOCK_ELEMS, GGMLType
from .v4_block_ref import V4Config, synth_weights

ARCH = "deepseek4"
_SCORE = {"softmax": 1, "sigmoid": 2, "sqrtsoftplus": 3}
_SCORE_INV = {v: k for k, v in _SCORE.items()}


@dataclass(frozen=True)
class Row:
    gguf: str                 # name in the file, "{L}" = block number
    key: str                  # key in the runtime's weight dictionary, "{P}" = "layers.<L>." (or "mtp.")
    kind: str                 # matrix | vector | experts | table
    when: str = "always"      # always | hashed | routed_bias | compressed | indexer


GLOBAL_ROWS = (
    Row("token_embd.weight", "embed", "matrix"),
    Row("output.weight", "head", "matrix"),
    Row("output_norm.weight", "norm", "vector"),
    Row("output_hc_fn.weight", "hc_head_fn", "matrix"),
    Row("output_hc_base.weight", "hc_head_base", "vector"),
    Row("output_hc_scale.weight", "hc_head_scale", "vector"),
)

LAYER_ROWS = (
    Row("blk.{L}.attn_sinks.weight", "{P}attn.attn_sink", "vector"),
    Row("blk.{L}.attn_q_a.weight", "{P}attn.wq_a", "matrix"),
    Row("blk.{L}.attn_q_a_norm.weight", "{P}attn.q_norm", "vector"),
    Row("blk.{L}.attn_q_b.weight", "{P}attn.wq_b", "matrix"),
    Row("blk.{L}.attn_kv.weight", "{P}attn.wkv", "matrix"),
    Row("blk.{L}.attn_kv_a_norm.weight", "{P}attn.kv_norm", "vector"),
    Row("blk.{L}.attn_output_a.weight", "{P}attn.wo_a", "matrix"),
    Row("blk.{L}.attn_output_b.weight", "{P}attn.wo_b", "matrix"),
    Row("blk.{L}.attn_norm.weight", "{P}attn_norm", "vector"),
    Row("blk.{L}.ffn_gate_inp.weight", "{P}ffn.gate", "matrix"),
    Row("blk.{L}.ffn_gate_tid2eid.weight", "{P}ffn.tid2eid", "table", "hashed"),
    Row("blk.{L}.exp_probs_b.bias", "{P}ffn.gate_bias", "vector", "routed_bias"),
    Row("blk.{L}.ffn_gate_exps.weight", "{P}ffn.experts.{E}.w1", "experts"),
    Row("blk.{L}.ffn_down_exps.weight", "{P}ffn.experts.{E}.w2", "experts"),
    Row("blk.{L}.ffn_up_exps.weight", "{P}ffn.experts.{E}.w3", "experts"),
    Row("blk.{L}.ffn_gate_shexp.weight", "{P}ffn.experts.shared.w1", "matrix"),
    Row("blk.{L}.ffn_down_shexp.weight", "{P}ffn.experts.shared.w2", "matrix"),
    Row("blk.{L}.ffn_up_shexp.weight", "{P}ffn.experts.shared.w3", "matrix"),
    Row("blk.{L}.ffn_norm.weight", "{P}ffn_norm", "vector"),
    Row("blk.{L}.hc_attn_fn.weight", "{P}hc_attn_fn", "matrix"),
    Row("blk.{L}.hc_attn_base.weight", "{P}hc_attn_base", "vector"),
    Row("blk.{L}.hc_attn_scale.weight", "{P}hc_attn_scale", "vector"),
    Row("blk.{L}.hc_ffn_fn.weight", "{P}hc_ffn_fn", "matrix"),
    Row("blk.{L}.hc_ffn_base.weight", "{P}hc_ffn_base", "vector"),
    Row("blk.{L}.hc_ffn_scale.weight", "{P}hc_ffn_scale", "vector"),
    Row("blk.{L}.attn_compressor_ape.weight", "{P}attn.compressor.ape", "matrix", "compressed"),
    Row("blk.{L}.attn_compressor_kv.weight", "{P}attn.compressor.wkv", "matrix", "compressed"),
    Row("blk.{L}.attn_compressor_gate.weight", "{P}attn.compressor.wgate", "matrix", "compressed"),
    Row("blk.{L}.attn_compressor_norm.weight", "{P}attn.compressor.norm", "vector", "compressed"),
    Row("blk.{L}.indexer.attn_q_b.weight", "{P}attn.indexer.wq_b", "matrix", "indexer"),
    Row("blk.{L}.indexer.proj.weight", "{P}attn.indexer.weights_proj", "matrix", "indexer"),
    Row("blk.{L}.indexer_compressor_ape.weight", "{P}attn.indexer.compressor.ape", "matrix", "indexer"),
    Row("blk.{L}.indexer_compressor_kv.weight", "{P}attn.indexer.compressor.wkv", "matrix", "indexer"),
    Row("blk.{L}.indexer_compressor_gate.weight", "{P}attn.indexer.compressor.wgate", "matrix", "indexer"),
    Row("blk.{L}.indexer_compressor_norm.weight", "{P}attn.indexer.compressor.norm", "vector", "indexer"),
)

# the multi-token-prediction block sits after the last layer (block number n_layers) with these extras
MTP_ROWS = (
    Row("blk.{L}.nextn.e_proj.weight", "mtp.e_proj", "matrix"),
    Row("blk.{L}.nextn.h_proj.weight", "mtp.h_proj", "matrix"),
    Row("blk.{L}.nextn.enorm.weight", "mtp.enorm", "vector"),
    Row("blk.{L}.nextn.hnorm.weight", "mtp.hnorm", "vector"),
    Row("blk.{L}.nextn.shared_head_norm.weight", "mtp.norm", "vector"),
    Row("blk.{L}.nextn.hc_head_fn.weight", "mtp.hc_head_fn", "matrix"),
    Row("blk.{L}.nextn.hc_head_base.weight", "mtp.hc_head_base", "vector"),
    Row("blk.{L}.nextn.hc_head_scale.weight", "mtp.hc_head_scale", "vector"),
)


@dataclass(frozen=True)
class Entry:
    gguf: str
    key: str
    kind: str
    expert: int | None = None


def _applies(row: Row, ratio: int, hashed: bool) -> bool:
    return {"always": True, "hashed": hashed, "routed_bias": not hashed, "compressed": ratio != 0,
            "indexer": ratio == 4}[row.when]


def expected_entries(cfg: V4Config) -> list[Entry]:
    """Every (file tensor, runtime key) pair a checkpoint of this shape must provide, experts expanded."""
    out = [Entry(r.gguf, r.key, r.kind) for r in GLOBAL_ROWS]
    blocks = [(i, f"layers.{i}.", ratio, i < cfg.n_hash_layers) for i, ratio in enumerate(cfg.compress_ratios)]
    if cfg.mtp:
        blocks.append((cfg.n_layers, "mtp.", 0, False))
    for layer, prefix, ratio, hashed in blocks:
        for r in LAYER_ROWS:
            if not _applies(r, ratio, hashed):
                continue
            name, key = r.gguf.replace("{L}", str(layer)), r.key.replace("{P}", prefix)
            if r.kind == "experts":
                out.extend(Entry(name, key.replace("{E}", str(e)), "experts", e) for e in range(cfg.n_experts))
            else:
                out.append(Entry(name, key, r.kind))
    if cfg.mtp:
        out.extend(Entry(r.gguf.replace("{L}", str(cfg.n_layers)), r.key, r.kind) for r in MTP_ROWS)
    return out


# ---------------------------------------------------------------------------------------------- metadata
def metadata(cfg: V4Config) -> dict[str, Any]:
    a = ARCH
    return {
        "general.architecture": a, "general.name": "deepseek-v4-shaped",
        f"{a}.vocab_size": cfg.vocab_size, f"{a}.embedding_length": cfg.dim, f"{a}.block_count": cfg.n_layers,
        f"{a}.attention.head_count": cfg.n_heads, f"{a}.attention.head_count_kv": 1,
        f"{a}.attention.key_length": cfg.head_dim, f"{a}.attention.value_length": cfg.head_dim,
        f"{a}.attention.q_lora_rank": cfg.q_lora_rank, f"{a}.attention.output_lora_rank": cfg.o_lora_rank,
        f"{a}.attention.output_group_count": cfg.o_groups, f"{a}.attention.sliding_window": cfg.window,
        f"{a}.attention.compress_ratios": list(cfg.compress_ratios),
        f"{a}.attention.compress_rope_freq_base": float(cfg.compress_rope_theta),
        f"{a}.attention.indexer.head_count": cfg.index_n_heads, f"{a}.attention.indexer.key_length": cfg.index_head_dim,
        f"{a}.attention.indexer.top_k": cfg.index_topk,
        f"{a}.attention.layer_norm_rms_epsilon": float(cfg.norm_eps),
        f"{a}.expert_count": cfg.n_experts, f"{a}.expert_used_count": cfg.n_activated,
        f"{a}.expert_shared_count": cfg.n_shared, f"{a}.expert_feed_forward_length": cfg.moe_inter,
        f"{a}.expert_weights_scale": float(cfg.route_scale), f"{a}.expert_gating_func": _SCORE[cfg.score_func],
        f"{a}.swiglu_limit": float(cfg.swiglu_limit), f"{a}.hash_layer_count": cfg.n_hash_layers,
        f"{a}.hyper_connection.count": cfg.hc_mult, f"{a}.hyper_connection.sinkhorn_iterations": cfg.hc_iters,
        f"{a}.hyper_connection.epsilon": float(cfg.hc_eps),
        f"{a}.rope.dimension_count": cfg.rope_head_dim, f"{a}.rope.freq_base": float(cfg.rope_theta),
        f"{a}.rope.scaling.factor": float(cfg.rope_factor),
        f"{a}.rope.scaling.original_context_length": cfg.original_seq_len, f"{a}.context_length": cfg.max_seq_len,
        f"{a}.nextn_predict_layers": 1 if cfg.mtp else 0,
    }


def config_from_metadata(md: dict[str, Any]) -> V4Config:
    a = str(md.get("general.architecture", ARCH))
    if a != ARCH:
        raise ValueError(f"not a {ARCH} checkpoint: general.architecture = {a!r}")

    def g(suffix: str, default=None):
        v = md.get(f"{a}.{suffix}", default)
        if v is None:
            raise KeyError(f"{a}.{suffix} is missing from the metadata")
        return v

    def fl(suffix: str, default=None) -> float:
        # floats are stored as 32-bit values: give back the shortest decimal that names the same 32-bit number
        return float(f"{float(g(suffix, default)):.7g}")

    d = V4Config()
    return V4Config(
        vocab_size=int(g("vocab_size")), dim=int(g("embedding_length")), n_layers=int(g("block_count")),
        n_heads=int(g("attention.head_count")), head_dim=int(g("attention.key_length")),
        rope_head_dim=int(g("rope.dimension_count")), q_lora_rank=int(g("attention.q_lora_rank")),
        o_groups=int(g("attention.output_group_count")), o_lora_rank=int(g("attention.output_lora_rank")),
        window=int(g("attention.sliding_window")), compress_ratios=tuple(int(x) for x in g("attention.compress_ratios")),
        index_n_heads=int(g("attention.indexer.head_count")), index_head_dim=int(g("attention.indexer.key_length")),
        index_topk=int(g("attention.indexer.top_k")), hc_mult=int(g("hyper_connection.count")),
        hc_iters=int(g("hyper_connection.sinkhorn_iterations", d.hc_iters)),
        hc_eps=fl("hyper_connection.epsilon", d.hc_eps), n_experts=int(g("expert_count")),
        n_activated=int(g("expert_used_count")), n_shared=int(g("expert_shared_count", 1)),
        moe_inter=int(g("expert_feed_forward_length")), n_hash_layers=int(g("hash_layer_count", 0)),
        score_func=_SCORE_INV.get(int(g("expert_gating_func", _SCORE[d.score_func])), d.score_func),
        route_scale=fl("expert_weights_scale", d.route_scale), swiglu_limit=fl("swiglu_limit", d.swiglu_limit),
        rope_theta=fl("rope.freq_base", d.rope_theta),
        compress_rope_theta=fl("attention.compress_rope_freq_base", d.compress_rope_theta),
        rope_factor=fl("rope.scaling.factor", 1.0),
        original_seq_len=int(g("rope.scaling.original_context_length", d.original_seq_len)),
        norm_eps=fl("attention.layer_norm_rms_epsilon", d.norm_eps), max_seq_len=int(g("context_length", d.max_seq_len)),
        mtp=int(g("nextn_predict_layers", 0)) > 0)


# ---------------------------------------------------------------------------------------------- validation
@dataclass
class Validation:
    missing: list[str] = field(default_factory=list)          # in the table, not in the file
    unmapped: list[str] = field(default_factory=list)         # in the file, not in the table
    shape_errors: list[str] = field(default_factory=list)
    entries: list[Entry] = field(default_factory=list)

    @property
    def ok(self) -> bool:
        return not (self.missing or self.unmapped or self.shape_errors)

    def summary(self) -> str:
        return (f"{len(self.entries)} mapped, {len(self.missing)} missing, {len(self.unmapped)} unmapped, "
                f"{len(self.shape_errors)} shape errors")


def _expected_shape(cfg: V4Config, e: Entry, like: dict[str, torch.Tensor]) -> tuple[int, ...]:
    s = tuple(like[e.key].shape)
    return (cfg.n_experts, *s) if e.kind == "experts" else s


def validate(tensors: dict[str, Any], cfg: V4Config) -> Validation:
    """``tensors``: name -> object with ``.shape`` (torch order).  Checks presence both ways and every shape against
    the runtime's own weight shapes for this config (taken from a synthetic weight set, so the two cannot drift)."""
    like = synth_weights(cfg)
    v = Validation(entries=expected_entries(cfg))
    seen = set()
    for e in v.entries:
        if e.gguf not in tensors:
            if e.gguf not in seen:
                v.missing.append(e.gguf)
            seen.add(e.gguf)
            continue
        if e.gguf in seen:
            continue
        seen.add(e.gguf)
        want, got = _expected_shape(cfg, e, like), tuple(int(x) for x in tensors[e.gguf].shape)
        if e.kind == "vector" and len(got) == 2 and got[0] == 1:
            got = got[1:]
        if want != got:
            v.shape_errors.append(f"{e.gguf}: file has {list(got)}, {e.key} wants {list(want)}")
    v.unmapped = sorted(n for n in tensors if n not in seen)
    return v


# ---------------------------------------------------------------------------------------------- write / read
def _file_type(kind: str, cols: int, matrix_type: GGMLType) -> GGMLType:
    if kind in ("vector", "table"):
        return GGMLType.F32
    return matrix_type if cols % BLOCK_ELEMS[matrix_type] == 0 else GGMLType.F16


def write_gguf(path: str, cfg: V4Config, weights: dict[str, torch.Tensor],
               matrix_type: GGMLType | str = GGMLType.F32) -> None:
    """Write ``weights`` (the block runtime's dictionary) as a ``deepseek4`` GGUF.  Matrices take ``matrix_type`` when
    their row length allows it (else F16); vectors and the token->expert table are F32."""
    mt = GGMLType[matrix_type] if isinstance(matrix_type, str) else GGMLType(matrix_type)
    out, done = [], set()
    for e in expected_entries(cfg):
        if e.gguf in done:
            continue
        done.add(e.gguf)
        if e.kind == "experts":
            head, tail = e.key.rsplit(f".experts.{e.expert}.", 1)
            w = torch.stack([weights[f"{head}.experts.{k}.{tail}"] for k in range(cfg.n_experts)])
        else:
            w = weights[e.key]
        w = w.float()
        shape = tuple(w.shape) if w.dim() > 1 else (1, w.shape[0])
        t = _file_type(e.kind, shape[-1], mt)
        raw = G.quantize(w.reshape(-1, shape[-1]), t)
        out.append((e.gguf, raw, t, shape if w.dim() > 1 else (w.shape[0],)))
    G.write_gguf(path, metadata(cfg), out)


def load(path: str, strict: bool = True) -> tuple[V4Config, dict[str, torch.Tensor]]:
    """Read a ``deepseek4`` checkpoint into (config, fp32 weight dictionary) for ``V4BlockRef``.  With ``strict`` every
    mismatch between file and table raises one error that lists them all."""
    return load_bundle(G.read_bundle(path), strict, path)


def load_bundle(bundle, strict: bool = True, path: str = "checkpoint") -> tuple[V4Config, dict[str, torch.Tensor]]:
    cfg = config_from_metadata(bundle.metadata)
    v = validate(bundle.tensors, cfg)
    if strict and not v.ok:
        lines = [f"missing {n}" for n in v.missing] + [f"unmapped {n}" for n in v.unmapped] + v.shape_errors
        raise ValueError(f"{path}: {v.summary()}\n  " + "\n  ".join(lines[:40]))
    like = synth_weights(cfg) if not strict else None
    w: dict[str, torch.Tensor] = {}
    cache: dict[str, torch.Tensor] = {}
    for e in v.entries:
        if e.gguf not in bundle.tensors:
            if like is not None:
                w[e.key] = like[e.key]
            continue
        if e.gguf not in cache:
            cache.clear()                      # one stacked expert tensor at a time
            cache[e.gguf] = bundle.dequantized(e.gguf)
        t = cache[e.gguf]
        if e.kind == "experts":
            t = t[e.expert]
        elif e.kind == "vector":
            t = t.reshape(-1)
        elif e.kind == "table":
            t = t.round().to(torch.int64)
        w[e.key] = t.clone() if e.kind == "experts" else t
    return cfg, w
