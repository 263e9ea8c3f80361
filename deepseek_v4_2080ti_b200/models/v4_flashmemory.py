"""Long-context decode for the DeepSeek-V4 CPU runtime: a shared learned retriever chooses the compressed entries every
indexer layer attends to, and the compressed rows live in a host pool with a small working set next to the model.

The two components exist on their own (``components/flashmemory.py``: scorer, ensemble, top-k, with sm_100a kernels;
``runtime/kv_swap.py``: pinned host pool, LRU working set, side-stream copies); this module is the wiring around the
V4 block runtime (``models/v4_block_ref.py``), as the reference's plugin wires them into its engine:

* Once per decode token, before the layers run: every retriever layer (its own ``wq_a / wq_b / q_norm / weights_proj``,
  loaded from ``retrievers.l<ID>.*``) builds index queries from the token's *embedding*, scores the indexer keys of one
  source layer (the first ratio-4 layer; its keys are shared by all retriever layers), the scores are combined by max
  or mean, and the best ``index_topk`` of the ``position // ratio`` finished entries are kept.
* Every ratio-4 layer then takes that one selection in place of its own indexer's (its indexer still appends its keys:
  the source layer's are what the retriever scores).  The prompt pass keeps the layers' own indexers.
* With the swap on, a ratio-4 layer no longer keeps its compressed rows: finished groups of ``chunk_entries`` rows go to
  the host pool, the selection is made resident (hits are free, misses evict the least recently used groups) and the
  attention reads ``[window ring | staged rows]``.  The newest, unfinished group stays in a small resident tail.

Reference behaviour: cpp_engine/engine/deepseek_v4_engine.cpp:9325-9378 (per-token scoring from the embedding row against
the source layer's indexer cache, ensemble, global top-k), :5813-5833 (layers write the global indices behind the
window), :5362-5640 (host pool and staging), docs/FLASHMEMORY_1M_CONTEXT.md (working-set sizing: at least
``index_topk`` slots).
"""
from __future__ import annotations

import torch

from ..components import flashmemory as fm
from ..runtime.kv_swap import KvSwapManager
from .v4_block_ref import V4BlockRef, V4Config


def synth_retriever_weights(cfg: V4Config, n_retrievers: int = 2, heads: int = 4, q_lora: int = 16, seed: int = 0) -> dict:
    """``retrievers.l<i>.{wq_a.weight,wq_b.weight,q_norm_weight,weights_proj.weight}`` of a random retriever."""
    g = torch.Generator().manual_seed(seed + 313)
    w = {}
    for i in range(n_retrievers):
        p = f"retrievers.l{i}."
        w[p + "wq_a.weight"] = torch.randn(q_lora, cfg.dim, generator=g) * 0.2
        w[p + "wq_b.weight"] = torch.randn(heads * fm.D, q_lora, generator=g) * 0.2
        w[p + "q_norm_weight"] = 1.0 + torch.randn(q_lora, generator=g) * 0.05
        w[p + "weights_proj.weight"] = torch.randn(heads, cfg.dim, generator=g) * 0.3
    return w


RETRIEVER_TENSORS = ("wq_a.weight", "wq_b.weight", "q_norm_weight", "weights_proj.weight")


def load_retrievers(path: str, hidden: int) -> dict:
    """Read a retriever checkpoint (one safetensors file, ``retrievers.l<ID>.*``; f32 / bf16 / f16) and check that every
    layer is complete and shaped for a model of width ``hidden`` with 128-wide index heads
    (cpp_engine/engine/deepseek_v4_engine.cpp:190-240)."""
    from ..formats.safetensors_io import SafetensorsFile
    f = SafetensorsFile(path)
    names = [k for k in f.keys() if k.startswith("retrievers.")]
    layers = sorted({k.split(".")[1] for k in names})
    if not layers:
        raise ValueError(f"{path}: no retrievers.l<ID>.* tensors")
    out = {}
    for l in layers:
        for suffix in RETRIEVER_TENSORS:
            k = f"retrievers.{l}.{suffix}"
            if k not in names:
                raise ValueError(f"{path}: missing {k}")
            out[k] = f.get(k).float()
        a, b = out[f"retrievers.{l}.wq_a.weight"], out[f"retrievers.{l}.wq_b.weight"]
        n, p = out[f"retrievers.{l}.q_norm_weight"], out[f"retrievers.{l}.weights_proj.weight"]
        heads = b.shape[0] // fm.D
        if a.shape[1] != hidden or b.shape != (heads * fm.D, a.shape[0]) or n.shape != (a.shape[0],) or p.shape != (heads, hidden):
            raise ValueError(f"{path}: retriever {l} does not fit a model of width {hidden}")
    return out


class CompressedRowStore:
    """Compressed KV rows of one layer, kept outside the layer: groups of ``chunk_entries`` rows in the swap manager's
    host pool, the unfinished newest group in a resident tail."""

    def __init__(self, capacity: int, chunk_entries: int, head_dim: int, device_chunks: int, device="cpu"):
        self.g, self.head_dim = int(chunk_entries), int(head_dim)
        n_chunks = (capacity + self.g - 1) // self.g
        self.swap = KvSwapManager(n_chunks, device_chunks, self.g, head_dim * 4, device=device)
        self.tail = torch.zeros(self.g, head_dim, device=self.swap.device)
        self.count = 0

    def reset(self) -> None:
        sw = self.swap
        self.swap = KvSwapManager(sw.host.shape[0], sw.dev.shape[0], self.g, self.head_dim * 4, device=sw.device)
        self.tail.zero_()
        self.count = 0

    def append(self, entry: int, row: torch.Tensor) -> None:
        if entry != self.count:
            raise RuntimeError("compressed rows arrive in order")
        self.tail[entry % self.g] = row.to(self.tail.device)
        self.count += 1
        if self.count % self.g == 0:
            self.swap.store(entry // self.g, self.tail.clone().view(torch.uint8).view(self.g, -1))

    def gather(self, entries: torch.Tensor) -> torch.Tensor:
        """Rows [len(entries), head_dim] of the named entries (-1: a zero row nobody attends to)."""
        e = entries.long()
        live = (e >= 0) & (e // self.g < self.count // self.g)            # in a finished group
        out = torch.zeros(e.numel(), self.head_dim, device=self.tail.device)
        if bool(live.any()):
            chunks = torch.unique(e[live] // self.g)
            slots = self.swap.ensure(chunks)
            slot_of = torch.full((int(chunks.max()) + 1,), -1, dtype=torch.long, device=slots.device)
            slot_of[chunks] = slots.long()
            staged = self.swap.dev.view(torch.float32).view(-1, self.g, self.head_dim)
            out[live] = staged[slot_of[e[live] // self.g], e[live] % self.g]
        tail = (e >= 0) & ~live
        if bool(tail.any()):
            if int(e[tail].max()) >= self.count:
                raise RuntimeError("entry not stored yet")
            out[tail] = self.tail[e[tail] % self.g]
        return out


class V4LongContextRuntime(V4BlockRef):
    """``V4BlockRef`` with the shared retriever (``retrievers`` given) and / or the swapped compressed rows
    (``swap_device_chunks > 0``).  Same ``forward`` / ``generate`` contract; ``snapshot`` is refused while rows live in
    the host pool."""

    def __init__(self, cfg: V4Config, weights: dict, retrievers: dict | None = None, use_max: bool = True,
                 swap_device_chunks: int = 0, chunk_entries: int = 4, device="cpu"):
        super().__init__(cfg, weights)
        self.indexed = [l for l in self.layers if l.ratio == 4]
        if not self.indexed:
            raise ValueError("no ratio-4 layer: nothing to retrieve or swap")
        self.src = self.indexed[0]
        self.retriever = None
        if retrievers:
            names = sorted({k.split(".")[1] for k in retrievers if k.startswith("retrievers.")})
            layers = []
            for n in names:
                p = f"retrievers.{n}."
                layers.append(fm.ScorerLayer(retrievers[p + "wq_a.weight"].float(), retrievers[p + "wq_b.weight"].float(),
                                             retrievers[p + "q_norm_weight"].float(), retrievers[p + "weights_proj.weight"].float(),
                                             keys=self.src.ikeys))
            inv = fm.yarn_inv_freqs(cfg.rope_head_dim, cfg.compress_rope_theta, cfg.rope_factor, cfg.original_seq_len)
            self.retriever = fm.FlashMemoryRetriever(layers, inv, chunk_tokens=4, keep=cfg.index_topk, use_max=use_max,
                                                     eps=cfg.norm_eps)
        self.stores: list[CompressedRowStore] = []
        if swap_device_chunks:
            need = min(cfg.index_topk, -(-cfg.max_seq_len // 4 // chunk_entries))
            if swap_device_chunks < need:
                raise ValueError(f"the working set must hold one step's selection: {need} groups")
            for l in self.indexed:
                l.store = CompressedRowStore(cfg.max_seq_len // 4, chunk_entries, cfg.head_dim, swap_device_chunks, device)
                self.stores.append(l.store)
        self.last_selection: torch.Tensor | None = None
        self.reset()

    def reset(self) -> None:
        for st in getattr(self, "stores", []):
            st.reset()
        super().reset()
        for l in getattr(self, "indexed", []):
            l.global_pick = None

    def snapshot(self) -> dict:
        if self.stores:
            raise RuntimeError("snapshots are not taken while compressed rows live in the host pool")
        return super().snapshot()

    def select(self, token: int, position: int) -> torch.Tensor:
        """Entry ids int64 [index_topk] (-1 padded) for the decode token ``token`` at ``position``."""
        r = self.retriever
        available = min(position // 4, self.src.ikeys.shape[0])
        keep = min(self.cfg.index_topk, available)
        pick = torch.full((self.cfg.index_topk,), -1, dtype=torch.long)
        if keep > 0:
            for l in r.layers:                                  # all retriever layers read the source layer's keys
                l.keys, l.n_chunks = self.src.ikeys, available
            ids, _ = r.select([self.w["embed"][token]] * len(r.layers), position)
            pick[:keep] = ids[:keep].long()
        return pick

    @torch.no_grad()
    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        ids = ids.reshape(-1).long()
        pick = None
        if self.retriever is not None and self.length > 0 and ids.numel() == 1:
            pick = self.select(int(ids[0]), self.length)
        self.last_selection = pick
        for l in self.indexed:
            l.global_pick = pick
        try:
            return super().forward(ids)
        finally:
            for l in self.indexed:
                l.global_pick = None

    def swap_stats(self) -> dict:
        tot: dict = {}
        for st in self.stores:
            for k, v in st.swap.stats().items():
                tot[k] = tot.get(k, 0) + v
        return tot
