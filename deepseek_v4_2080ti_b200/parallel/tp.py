"""Tensor-parallel communicator.

``TPComm`` is the NCCL baseline (what the reference does with ``all_reduce_half`` after every
row-parallel projection, cpp_engine/engine/qwen_engine.cpp:2010-2037, and the packed arg-max merge,
cpp_engine/backends/cuda/collective/tp_comm.cpp:345-364).  The fused paths replace ``all_reduce``
with in-kernel peer-memory reductions; they plug in through the same interface.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def init_distributed(backend: str | None = None) -> tuple[int, int, int]:
    """Initialise torch.distributed from the torchrun environment. Returns (rank, world, local_rank)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local)
            dist.init_process_group(backend, rank=rank, world_size=world, device_id=torch.device("cuda", local))
        else:
            dist.init_process_group(backend, rank=rank, world_size=world)
    return rank, world, local


class TPComm:
    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.bytes_reduced = 0

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
            self.bytes_reduced += t.numel() * t.element_size()
        return t

    def argmax_merge(self, idx: torch.Tensor, val: torch.Tensor) -> torch.Tensor:
        """Global arg-max from per-rank (index, value) winners over vocab shards; ties go to the lower id."""
        if self.world == 1:
            return idx
        packed = torch.stack([val.float(), idx.float()], -1).contiguous()       # ids < 2^24 are exact in fp32
        gathered = torch.empty(self.world, *packed.shape, dtype=packed.dtype, device=packed.device)
        dist.all_gather_into_tensor(gathered, packed, group=self.group)
        vals, ids = gathered[..., 0], gathered[..., 1]
        best = vals.max(0, keepdim=True).values
        cand = torch.where(vals == best, ids, torch.full_like(ids, float("inf")))
        return cand.min(0).values.to(torch.int32)

    def barrier(self) -> None:
        if self.world > 1:
            dist.barrier(group=self.group)
