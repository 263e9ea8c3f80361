"""Model-family registry for GGUF checkpoints: detect the family from ``general.architecture``, parse its
hyper-parameters, check the tensor inventory against the family's naming, report which tensor types the runtime can
execute, and plan placement on a B200 box (everything resident; experts sharded by range).

Reference behaviour: the MoE spec registry (src/components/moe/spec.py:80-98, registry.py:10-47), the capability table
(capability.py:7-63) and the placement decisions (placement.py:9-56)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

from ..formats.gguf import BLOCK_BYTES, BLOCK_ELEMS, GGMLType

# GGUF types the tensor-core GEMM decodes in registers, and plain types every loader reads
GEMM_DECODED = {GGMLType.Q8_0, GGMLType.Q4_K, GGMLType.Q5_K, GGMLType.Q6_K, GGMLType.Q3_K, GGMLType.Q2_K, GGMLType.IQ1_M,
                GGMLType.IQ2_XXS, GGMLType.IQ2_XS, GGMLType.IQ3_XXS, GGMLType.IQ4_XS}
PLAIN = {GGMLType.F32, GGMLType.F16, GGMLType.BF16}


@dataclass(frozen=True)
class HardwareProfile:
    gpu_count: int = 8
    gpu_memory_gib: float = 180.0
    name: str = "8xB200"

    @property
    def per_gpu_bytes(self) -> int:
        return int(self.gpu_memory_gib * (1 << 30))


@dataclass
class PlacementDecision:
    name: str
    status: str                 # candidate | rejected
    reason: str
    bytes_per_gpu: int


@dataclass
class ValidationReport:
    architecture: str
    ok: bool
    missing: list[str] = field(default_factory=list)
    unexpected: list[str] = field(default_factory=list)
    by_type: dict[str, int] = field(default_factory=dict)        # type name -> bytes
    unsupported: dict[str, str] = field(default_factory=dict)    # tensor -> reason
    total_bytes: int = 0
    routed_bytes: int = 0


@dataclass
class ModelSpec:
    architecture: str
    display_name: str
    parse_params: Callable[[dict[str, Any], dict | None], Any]
    global_tensors: tuple[str, ...]
    layer_tensors: Callable[[Any, int], tuple[str, ...]]         # (params, layer) -> suffixes after ``blk.N.``
    n_layers: Callable[[Any], int]
    routed_suffixes: tuple[str, ...]
    build_runtime: Callable[..., Any] | None = None
    optional_suffixes: tuple[str, ...] = ()                     # present in some checkpoints, not needed by the runtime

    def expected_names(self, params) -> list[str]:
        out = list(self.global_tensors)
        for i in range(self.n_layers(params)):
            out += [f"blk.{i}.{s}" for s in self.layer_tensors(params, i)]
        return out

    def validate(self, bundle) -> ValidationReport:
        params = self.parse_params(bundle.metadata, bundle.tensors)
        want = set(self.expected_names(params))
        have = set(bundle.tensors)
        extra = sorted(n for n in have - want if not n.endswith(self.optional_suffixes or ("\0",)))
        rep = ValidationReport(self.architecture, True, sorted(want - have), extra)
        for name, ti in bundle.tensors.items():
            rep.by_type[ti.ggml_type.name] = rep.by_type.get(ti.ggml_type.name, 0) + ti.nbytes
            rep.total_bytes += ti.nbytes
            if any(name.endswith(s) for s in self.routed_suffixes):
                rep.routed_bytes += ti.nbytes
            status, why = capability_status(ti.ggml_type, two_d=len(ti.shape) >= 2)
            if status != "supported":
                rep.unsupported[name] = why
        rep.ok = not rep.missing and not rep.unsupported
        return rep

    def placement(self, report: ValidationReport, hw: HardwareProfile = HardwareProfile(), reserve_fraction: float = 0.15
                  ) -> list[PlacementDecision]:
        """Experts sharded by range over the GPUs, everything else sharded or replicated (counted as replicated: the
        upper bound).  The reference's host-staged expert placement is not needed when this fits."""
        shared = report.total_bytes - report.routed_bytes
        per_gpu = shared + (report.routed_bytes + hw.gpu_count - 1) // hw.gpu_count
        usable = int(hw.per_gpu_bytes * (1.0 - reserve_fraction))
        ok = per_gpu <= usable
        out = [PlacementDecision("all_device_resident", "candidate" if ok else "rejected",
                                 f"{per_gpu} bytes/GPU {'within' if ok else 'above'} the budget of {usable} bytes/GPU on {hw.name}",
                                 per_gpu)]
        if not ok:
            stages = 2
            out.append(PlacementDecision("layer_pipeline", "candidate",
                                         f"{stages} pipeline stages halve the resident layers per GPU group", per_gpu // stages))
        return out


def capability_status(t: GGMLType, two_d: bool = True) -> tuple[str, str]:
    t = GGMLType(t)
    if t in PLAIN:
        return "supported", "plain tensor"
    if t in GEMM_DECODED:
        return "supported", f"{t.name} blocks are decoded inside the tensor-core GEMM"
    if t in BLOCK_BYTES:
        return "deferred", f"{t.name} is readable (header and block size known) but has no GEMM decode path"
    return "unsupported", f"unknown GGUF tensor type {int(t)}"


# ---------------------------------------------------------------------------------------------- families
def _minimax_params(md, tensors):
    from .gqa_moe import GqaMoeConfig
    return GqaMoeConfig.from_metadata(md, tensors)


def _minimax_runtime(bundle, device="cuda", rank=0, world=1, comm=None, **kw):
    from . import gqa_moe as gm
    cfg = gm.GqaMoeConfig.from_metadata(bundle.metadata, bundle.tensors)
    w = gm.GqaMoeGpuWeights(cfg, gm.TensorStore(bundle), device, rank, world)
    return cfg, gm.GqaMoeRuntime(cfg, w, comm=comm, **kw)


class _MlaSlotAdapter:
    """The one-sequence MLA runtime behind the slot interface the GGUF drivers use (allocate / prefill / decode / free)."""
    single_sequence = True

    def __init__(self, rt):
        self.rt = rt
        self.cfg = getattr(rt, "cfg", None)               # front ends read the vocabulary size from it
        from ..ops import basic
        self._argmax = basic.argmax

    def allocate(self) -> int:
        self.rt.reset()
        return 0

    def free(self, slot: int) -> None:
        self.rt.reset()

    def prefill(self, slot: int, ids, chunk: int = 2048):
        logits = None
        for s in range(0, ids.numel(), chunk):
            logits = self.rt.forward(ids[s:s + chunk])
        return self._argmax(logits[-1:])

    def decode(self, slots, ids):
        return self._argmax(self.rt.forward(ids)[-1:])


def _glm_params(md, tensors):
    from .mla_gguf import config_from_metadata
    return config_from_metadata(md, tensors)


def _glm_runtime(bundle, device="cuda", rank=0, world=1, comm=None, max_slots=1, max_context=4096, **kw):
    from . import mla_gguf as mg
    from . import mla_moe_gpu as mm
    from .gqa_moe import TensorStore
    cfg = mg.config_from_metadata(bundle.metadata, bundle.tensors)
    per = cfg.num_experts // world
    state = mg.read_state(TensorStore(bundle), cfg, device, expert_range=(rank * per, (rank + 1) * per))
    w = mm.MlaMoeGpuWeights(cfg, state, device, rank, world)
    if max_slots > 1:       # several resident sequences: one page pool, batched decode
        return cfg, mm.MlaMoeBatchRuntime(cfg, w, max_slots=max_slots, max_context=max_context, comm=comm, **kw)
    return cfg, _MlaSlotAdapter(mm.MlaMoeGpuRuntime(cfg, w, max_context=max_context, comm=comm, **kw))


def _glm_layer_tensors(cfg, i):
    from .mla_gguf import layer_suffixes
    return layer_suffixes(cfg, i)


MINIMAX_LAYER = ("attn_norm.weight", "ffn_norm.weight", "attn_q.weight", "attn_k.weight", "attn_v.weight", "attn_output.weight",
                 "attn_q_norm.weight", "attn_k_norm.weight", "ffn_gate_inp.weight", "exp_probs_b.bias", "ffn_gate_exps.weight",
                 "ffn_up_exps.weight", "ffn_down_exps.weight")

_REGISTRY: dict[str, ModelSpec] = {}


def register(spec: ModelSpec) -> None:
    _REGISTRY[spec.architecture] = spec


def detect(bundle) -> ModelSpec:
    arch = str(bundle.metadata.get("general.architecture", ""))
    if arch not in _REGISTRY:
        raise KeyError(f"no model family registered for GGUF architecture {arch!r} (known: {sorted(_REGISTRY)})")
    return _REGISTRY[arch]


def architectures() -> list[str]:
    return sorted(_REGISTRY)


register(ModelSpec(
    architecture="minimax-m2", display_name="MiniMax-M2 (GQA + routed experts)", parse_params=_minimax_params,
    global_tensors=("token_embd.weight", "output.weight", "output_norm.weight"),
    layer_tensors=lambda p, i: MINIMAX_LAYER, n_layers=lambda p: p.n_layers,
    routed_suffixes=("ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight"), build_runtime=_minimax_runtime))

register(ModelSpec(
    architecture="glm-dsa", display_name="GLM-DSA (MLA + sparse indexer + routed experts)", parse_params=_glm_params,
    global_tensors=("token_embd.weight", "output.weight", "output_norm.weight"), layer_tensors=_glm_layer_tensors,
    n_layers=lambda p: p.num_layers + p.mtp_layers,
    routed_suffixes=("ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight"), build_runtime=_glm_runtime,
    optional_suffixes=("indexer.k_norm.bias", "nextn.shared_head_norm.weight")))


# ---- DeepSeek-V4 (window ring + compressor + hash routing + hyper-connections): served by the fp32 block runtime on
# the host; the file's tensors are dequantised at load.  One sequence, one rank.
def _v4_params(md, tensors):
    from .v4_gguf import config_from_metadata
    return config_from_metadata(md)


def _v4_layer_tensors(cfg, i):
    from . import v4_gguf as vg
    if i < cfg.n_layers:
        ratio, hashed, rows = cfg.compress_ratios[i], i < cfg.n_hash_layers, vg.LAYER_ROWS
    else:
        ratio, hashed, rows = 0, False, vg.LAYER_ROWS + vg.MTP_ROWS
    return tuple(r.gguf.split("{L}.", 1)[1] for r in rows if vg._applies(r, ratio, hashed))


class _V4HostAdapter:
    """The block runtime behind the slot interface of the GGUF drivers; token ids come back on ``device``."""
    single_sequence = True

    def __init__(self, rt, device):
        self.rt, self.device, self.cfg = rt, device, rt.cfg

    def allocate(self) -> int:
        self.rt.reset()
        return 0

    def free(self, slot: int) -> None:
        self.rt.reset()

    def _tok(self, logits):
        import torch
        return torch.tensor([int(logits[-1].argmax())], dtype=torch.int64, device=self.device)

    def prefill(self, slot: int, ids, chunk: int = 0):
        return self._tok(self.rt.forward(ids.detach().cpu()))

    def decode(self, slots, ids):
        return self._tok(self.rt.forward(ids.detach().cpu()))

    def stats(self) -> dict:
        swap = getattr(self.rt, "swap_stats", None)
        return {"kv_swap_" + k: v for k, v in swap().items()} if callable(swap) else {}


class _V4SpecHostAdapter(_V4HostAdapter):
    """The block runtime with the DSpark block drafter in front of it (``models/v4_dspark_ref.py``): ``decode`` hands out
    one committed token per call and runs a new draft / verify round when the committed ones are used up.  Greedy: the
    tokens are the plain runtime's tokens."""

    def __init__(self, loop, device):
        super().__init__(loop.t, device)
        self.loop, self.stream, self.pos = loop, [], 0

    def _one(self, tok: int):
        import torch
        return torch.tensor([tok], dtype=torch.int64, device=self.device)

    def prefill(self, slot: int, ids, chunk: int = 0):
        self.stream, self.pos = [self.loop.prefill(ids.detach().cpu())], 1
        return self._one(self.stream[0])

    def decode(self, slots, ids):
        while self.pos >= len(self.stream):
            toks, _ = self.loop.step()                    # [the pending token, accepted drafts ...]; a new one is pending
            self.stream += toks[1:] + [self.loop.committed]
        self.pos += 1
        return self._one(self.stream[self.pos - 1])

    def stats(self) -> dict:
        lp = self.loop
        return {"spec_rounds": lp.rounds, "spec_drafted": lp.drafted, "spec_accepted": lp.accepted, "target_steps": lp.target_steps}


def _v4_runtime(bundle, device="cpu", rank=0, world=1, comm=None, **kw):
    """Long-context options, as keywords or through the environment switches the reference's engine reads
    (docs/FLASHMEMORY_1M_CONTEXT.md there): ``flashmemory`` / ``POCKETLLM_GGUF_FLASHMEMORY_CKPT`` (retriever checkpoint;
    ensemble ``POCKETLLM_GGUF_FLASHMEMORY_ENSEMBLE`` = max | mean) and ``kv_swap_chunks`` /
    ``POCKETLLM_GGUF_KV_SWAP=1`` + ``POCKETLLM_GGUF_KV_SWAP_GPU_CHUNKS`` (working-set groups of compressed rows).
    Speculation: ``dspark`` / ``POCKETLLM_GGUF_DSPARK_CKPT`` (drafter file or "synthetic"), ``dspark_block``, ``spec_gate``."""
    import os
    from . import v4_gguf as vg
    from .v4_block_ref import V4BlockRef
    if world != 1:
        raise ValueError("the deepseek4 block runtime is single-rank (fp32 on the host)")
    cfg, weights = vg.load_bundle(bundle)
    ckpt = kw.get("flashmemory") or os.environ.get("POCKETLLM_GGUF_FLASHMEMORY_CKPT")
    chunks = int(kw.get("kv_swap_chunks") or (os.environ.get("POCKETLLM_GGUF_KV_SWAP_GPU_CHUNKS", "512")
                                              if os.environ.get("POCKETLLM_GGUF_KV_SWAP", "0") == "1" else 0))
    if ckpt or chunks:
        from . import v4_flashmemory as lc
        ensemble = str(kw.get("flashmemory_ensemble") or os.environ.get("POCKETLLM_GGUF_FLASHMEMORY_ENSEMBLE", "max"))
        if ensemble not in ("max", "mean"):
            raise ValueError("the retriever ensemble is 'max' or 'mean'")
        rt = lc.V4LongContextRuntime(cfg, weights, retrievers=lc.load_retrievers(ckpt, cfg.dim) if ckpt else None,
                                     use_max=ensemble == "max", swap_device_chunks=chunks,
                                     chunk_entries=int(kw.get("kv_swap_chunk_entries", 4)))
        return cfg, _V4HostAdapter(rt, device)
    drafter = kw.get("dspark") or os.environ.get("POCKETLLM_GGUF_DSPARK_CKPT")
    if drafter:
        # ``dspark``: a safetensors file of ``dspark.*`` tensors (metadata ``target_layer_ids``: "1,2"), or "synthetic"
        from ..components.spec_gate import SpecGate
        from . import v4_dspark_ref as vd
        block = int(kw.get("dspark_block", 4))
        if drafter == "synthetic":
            layer_ids = tuple(sorted({max(0, cfg.n_layers // 2 - 1), cfg.n_layers - 1}))
            dw = vd.synth_dspark_weights(cfg, n_stages=2, n_target=len(layer_ids), seed=0)
        else:
            dw, layer_ids = vd.load_dspark_weights(drafter, cfg, kw.get("dspark_target_layers"))
        gate = SpecGate.from_env(block) if str(kw.get("spec_gate", "0")) in ("1", "true") else None
        loop = vd.DSparkLoop(vd.DSparkRef(V4BlockRef(cfg, weights), dw, layer_ids, block=block), gate)
        return cfg, _V4SpecHostAdapter(loop, device)
    return cfg, _V4HostAdapter(V4BlockRef(cfg, weights), device)


register(ModelSpec(
    architecture="deepseek4", display_name="DeepSeek-V4 (compressed sparse attention + hyper-connections, host fp32 runtime)",
    parse_params=_v4_params,
    global_tensors=("token_embd.weight", "output.weight", "output_norm.weight", "output_hc_fn.weight",
                    "output_hc_base.weight", "output_hc_scale.weight"),
    layer_tensors=_v4_layer_tensors, n_layers=lambda p: p.n_layers + (1 if p.mtp else 0),
    routed_suffixes=("ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight"), build_runtime=_v4_runtime))
