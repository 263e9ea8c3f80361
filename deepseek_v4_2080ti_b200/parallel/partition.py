"""Partition policies: which rank owns which part of which checkpoint tensor.

A policy is a grid (pipeline stages x tensor/expert-parallel ranks per stage) plus name-based shard rules:
``column_parallel`` (split the output rows), ``row_parallel`` (split the input columns; block-quantised formats on
whole blocks), ``expert_owned`` (contiguous expert ranges), ``vocab_parallel``, ``replicated``; layers are owned by the
stage that holds them.  The same rules serve every loader (safetensors, GGUF, synthetic), so the per-rank layout does
not depend on the checkpoint format, and loaders can ask for the slice of a tensor *before* reading it.

Policies: ``tp`` (one stage, every rank a TP/EP rank: the reference's ``legacy`` / ``baseline_4gpu``), ``layer_pp``
(contiguous layer ranges per stage, TP/EP inside a stage: the reference's ``layer_pp_4gpu`` generalised).
Reference behaviour: src/models/deepseek_v4/partition.py:61-67 (policies), :102-198 (rule kinds, shard shapes),
:241-291 (layer owner), :305+ (layout log)."""
from __future__ import annotations

import re
from dataclasses import dataclass

from .pp import PipelineLayout, split_layers

POLICIES = ("tp", "layer_pp")

# (regex on the tensor name, rule kind); first match wins.  Names follow this package's MLA family checkpoints and the
# Qwen-style hybrid checkpoints.
_RULES: list[tuple[re.Pattern, str]] = [(re.compile(p), k) for p, k in [
    (r"\.experts\.\d+\.", "expert_owned"),
    (r"(^|\.)embed(_tokens)?\.weight$", "vocab_parallel"),
    (r"(^|\.)(head|lm_head)\.weight$", "vocab_parallel"),
    (r"\.indexer\.", "replicated"),                                   # small; every rank scores with all index heads
    (r"\.(wq_b|wq|wkv_b|q_proj|k_proj|v_proj|in_proj_qkv|in_proj_z|in_proj_a|in_proj_b)\.(weight|weight_scale_inv|scale)$", "column_parallel"),
    (r"\.(w1|w3|gate_proj|up_proj)\.(weight|weight_scale_inv|scale)$", "column_parallel"),
    (r"\.(wo|o_proj|out_proj|w2|down_proj)\.(weight|weight_scale_inv|scale)$", "row_parallel"),
    (r"\.(A_log|dt_bias|conv1d\.weight)$", "column_parallel"),
    (r"\.attn_sink$", "column_parallel"),
]]


def normalize_policy(policy: str | None) -> str:
    policy = {"legacy": "tp", "baseline_4gpu": "tp", "layer_pp_4gpu": "layer_pp", None: "tp"}.get(policy, policy)
    if policy not in POLICIES:
        raise ValueError(f"unsupported partition policy {policy!r}; expected one of {POLICIES}")
    return policy


def rule_kind(name: str) -> str:
    for pat, kind in _RULES:
        if pat.search(name):
            return kind
    return "replicated"


def layer_of(name: str) -> int | None:
    m = re.search(r"(?:^|\.)layers\.(\d+)\.", name)
    return int(m.group(1)) if m else None


def expert_of(name: str) -> int | None:
    m = re.search(r"\.experts\.(\d+)\.", name)
    return int(m.group(1)) if m and "shared_experts" not in name else None


@dataclass
class Partition:
    policy: str
    rank: int
    world: int
    n_layers: int
    n_experts: int = 0
    stages: int = 1
    layer_weights: list[float] | None = None

    def __post_init__(self):
        self.policy = normalize_policy(self.policy)
        if self.policy == "tp":
            self.stages = 1
        self.layout = PipelineLayout(self.rank, self.world, self.stages)
        self.cuts = split_layers(self.n_layers, self.stages, self.layer_weights)
        if self.n_experts and self.n_experts % self.layout.tp:
            raise ValueError(f"{self.n_experts} experts do not divide over {self.layout.tp} ranks")

    # ---- ownership
    @property
    def layer_range(self) -> tuple[int, int]:
        return self.cuts[self.layout.stage]

    def stage_of_layer(self, layer: int) -> int:
        for s, (lo, hi) in enumerate(self.cuts):
            if lo <= layer < hi:
                return s
        raise ValueError(f"layer {layer} out of range")

    @property
    def expert_range(self) -> tuple[int, int]:
        per = self.n_experts // self.layout.tp if self.n_experts else 0
        return self.layout.tp_rank * per, (self.layout.tp_rank + 1) * per

    def owns(self, name: str) -> bool:
        """Does this rank need any part of the tensor?  (Checkpoint key filter: skip the read otherwise.)"""
        layer = layer_of(name)
        if layer is not None:
            lo, hi = self.layer_range
            if not (lo <= layer < hi):
                return False
        elif self.stages > 1:
            first, last = self.layout.is_first, self.layout.is_last
            if re.search(r"(^|\.)embed(_tokens)?\.weight$", name):
                return first
            if re.search(r"(^|\.)(head|lm_head|norm)\.weight$", name) or name.startswith("mtp."):
                return last
        e = expert_of(name)
        if e is not None:
            lo, hi = self.expert_range
            return lo <= e < hi
        return True

    def shard(self, name: str, shape: tuple[int, ...], block: int = 1) -> tuple[int | None, int, int]:
        """(dim, start, size) of this rank's slice, or (None, 0, 0) for a whole tensor.  ``block``: elements per
        quantisation block along the input dimension (row-parallel slices must hold whole blocks)."""
        kind = rule_kind(name)
        tpw, tpr = self.layout.tp, self.layout.tp_rank
        if tpw == 1 or kind in ("replicated", "expert_owned"):
            return None, 0, 0
        if kind == "vocab_parallel":
            per = (shape[0] + tpw - 1) // tpw
            lo = min(shape[0], tpr * per)
            return 0, lo, min(shape[0], lo + per) - lo
        dim = 0 if kind == "column_parallel" or len(shape) == 1 else 1
        if shape[dim] % tpw:
            raise ValueError(f"{name}: dimension {dim} of {shape} does not divide over {tpw} ranks")
        per = shape[dim] // tpw
        if dim == 1 and per % block:
            raise ValueError(f"{name}: a row-parallel slice of {per} columns splits a {block}-wide quantisation block")
        return dim, tpr * per, per

    def describe(self) -> str:
        lo, hi = self.layer_range
        e = f" experts [{self.expert_range[0]}, {self.expert_range[1]})" if self.n_experts else ""
        return (f"partition policy={self.policy} rank={self.rank}/{self.world} stage={self.layout.stage}/{self.stages} "
                f"tp_rank={self.layout.tp_rank}/{self.layout.tp} layers [{lo}, {hi}){e}")
