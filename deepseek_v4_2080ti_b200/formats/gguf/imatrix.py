"""Importance matrices of routed experts: per (layer, projection, expert) the sum of squared input activations per
input channel and the number of rows seen, in the GGUF layout llama.cpp's quantiser reads:
``<tensor>.in_sum2`` F32 [experts, width] and ``<tensor>.counts`` F32 [experts, 1], metadata ``general.type =
"imatrix"``, ``imatrix.datasets``, ``imatrix.chunk_size``, ``imatrix.chunk_count``.

The collector takes the expert-sorted activation rows that the grouped GEMM consumes (``observe_sorted``: rows plus the
per-expert offsets, reduced on the device in one segmented sum) or one expert's rows (``observe``); files from several
ranks or runs are summed by ``merge_imatrix_files``.

Reference behaviour: src/loader/gguf/imatrix.py:46-136 (collector), :179-240 (merge), :292+ (writer).
"""
from __future__ import annotations

import math
import os
import threading
from typing import Sequence

import torch

from .constants import GGMLType
from .reader import read_bundle
from .writer import write_gguf


def rank_output_path(path: str, rank: int | None = None, world: int | None = None) -> str:
    """``{rank}`` placeholders are filled in; otherwise multi-rank runs get ``.rankN`` before the extension."""
    rank = int(os.environ.get("RANK", "0")) if rank is None else rank
    world = int(os.environ.get("WORLD_SIZE", "1")) if world is None else world
    if "{rank}" in path:
        return path.format(rank=rank)
    if world <= 1:
        return path
    root, ext = os.path.splitext(path)
    return f"{root}.rank{rank}{ext or '.gguf'}"


class RoutedIMatrixCollector:
    def __init__(self, n_experts: int, dataset: str = "runtime_capture", chunk_size: int = 512,
                 layers: set[int] | None = None, roles: set[str] | None = None):
        self.n_experts, self.dataset, self.chunk_size = n_experts, dataset, max(1, chunk_size)
        self.layers, self.roles = layers, roles
        self._sum2: dict[str, torch.Tensor] = {}
        self._counts: dict[str, torch.Tensor] = {}
        self._lock = threading.Lock()

    def should_capture(self, layer: int, role: str) -> bool:
        return (self.layers is None or layer in self.layers) and (self.roles is None or role in self.roles)

    def _slot(self, layer: int, role: str, width: int, device) -> str:
        name = f"blk.{int(layer)}.{role}.weight"
        if name not in self._sum2:
            self._sum2[name] = torch.zeros(self.n_experts, width, dtype=torch.float32, device=device)
            self._counts[name] = torch.zeros(self.n_experts, dtype=torch.float32, device=device)
        elif self._sum2[name].shape[1] != width:
            raise ValueError(f"imatrix width mismatch for {name}: {self._sum2[name].shape[1]} vs {width}")
        return name

    def observe(self, layer: int, expert: int, role: str, x: torch.Tensor) -> None:
        """``x``: [..., width] inputs of one expert's projection ``role`` (e.g. ``ffn_gate_exps``)."""
        if not self.should_capture(layer, role) or not (0 <= expert < self.n_experts) or x.numel() == 0:
            return
        rows = x.detach().reshape(-1, x.shape[-1]).float()
        with self._lock:
            name = self._slot(layer, role, rows.shape[1], rows.device)
            self._sum2[name][expert] += (rows * rows).sum(0)
            self._counts[name][expert] += rows.shape[0]

    def observe_sorted(self, layer: int, role: str, x_sorted: torch.Tensor, offsets: torch.Tensor, expert_lo: int = 0) -> None:
        """Expert-sorted rows [R, width] with ``offsets`` int [E_local + 1] (rows of local expert e are
        ``offsets[e]:offsets[e+1]``; rows past ``offsets[-1]`` are padding)."""
        if not self.should_capture(layer, role):
            return
        rows = x_sorted.detach().float()
        off = offsets.to(torch.int64)
        e_local = off.numel() - 1
        r = torch.arange(rows.shape[0], device=rows.device)
        seg = torch.bucketize(r, off[1:], right=True)                     # local expert of each row; >= e_local: padding
        valid = seg < e_local
        with self._lock:
            name = self._slot(layer, role, rows.shape[1], rows.device)
            idx = (seg[valid] + expert_lo).clamp_max(self.n_experts - 1)
            self._sum2[name].index_add_(0, idx, rows[valid] ** 2)
            self._counts[name].index_add_(0, idx, torch.ones_like(idx, dtype=torch.float32))

    def entries(self) -> list[tuple[str, torch.Tensor, torch.Tensor]]:
        with self._lock:
            return sorted((n, self._sum2[n].cpu().clone(), self._counts[n].cpu().clone()) for n in self._sum2)

    def save(self, path: str) -> dict:
        ents = self.entries()
        if not ents:
            return {"entries": 0}
        return write_imatrix(path, ents, self.dataset, self.chunk_size)


def write_imatrix(path: str, entries: Sequence[tuple[str, torch.Tensor, torch.Tensor]], dataset: str, chunk_size: int) -> dict:
    max_count = max(float(c.max()) for _, _, c in entries)
    chunk_count = int(math.ceil(max_count / chunk_size)) if max_count > 0 else 0
    tensors = []
    for name, sum2, counts in entries:
        e, width = sum2.shape
        if counts.shape != (e,):
            raise ValueError(f"bad imatrix counts for {name}")
        tensors.append((f"{name}.in_sum2", sum2.float().contiguous().view(torch.uint8), GGMLType.F32, (e, width)))
        tensors.append((f"{name}.counts", counts.float().reshape(e, 1).contiguous().view(torch.uint8), GGMLType.F32, (e, 1)))
    meta = {"general.type": "imatrix", "imatrix.datasets": [dataset], "imatrix.chunk_count": chunk_count,
            "imatrix.chunk_size": int(chunk_size)}
    tmp = path + ".tmp"
    os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    write_gguf(tmp, meta, tensors, alignment=32)
    os.replace(tmp, path)
    return {"entries": len(entries), "chunk_count": chunk_count, "total_counts": sum(float(c.sum()) for _, _, c in entries)}


def read_imatrix(path: str) -> tuple[dict[str, tuple[torch.Tensor, torch.Tensor]], dict]:
    b = read_bundle(path)
    if b.metadata.get("general.type") != "imatrix":
        raise ValueError(f"{path} is not an imatrix GGUF")
    out = {}
    for name in sorted(n for n in b.tensors if n.endswith(".in_sum2")):
        base = name[:-len(".in_sum2")]
        if base + ".counts" not in b.tensors:
            raise ValueError(f"{path} is missing {base}.counts")
        sum2 = b.dequantized(name).float()
        counts = b.dequantized(base + ".counts").float().reshape(-1)
        if sum2.dim() != 2 or sum2.shape[0] != counts.shape[0]:
            raise ValueError(f"expert count mismatch for {base}: {tuple(sum2.shape)} vs {tuple(counts.shape)}")
        out[base] = (sum2, counts)
    return out, b.metadata


def merge_imatrix_files(inputs: Sequence[str], output_path: str, dataset: str = "runtime_capture_merged",
                        chunk_size: int | None = None) -> dict:
    if not inputs:
        raise ValueError("at least one imatrix input is required")
    merged: dict[str, tuple[torch.Tensor, torch.Tensor]] = {}
    for path in inputs:
        ents, meta = read_imatrix(path)
        if chunk_size is None and meta.get("imatrix.chunk_size") is not None:
            chunk_size = int(meta["imatrix.chunk_size"])
        for base, (s2, c) in ents.items():
            if base in merged:
                if merged[base][0].shape != s2.shape:
                    raise ValueError(f"shape mismatch while merging {base}")
                merged[base] = (merged[base][0] + s2, merged[base][1] + c)
            else:
                merged[base] = (s2.clone(), c.clone())
    if not merged:
        raise ValueError("no imatrix entries found")
    return write_imatrix(output_path, [(n, *merged[n]) for n in sorted(merged)], dataset, int(chunk_size or 512))
