"""Layer pipeline over point-to-point transfers (NCCL send/recv on NVLink; gloo on CPU for the tests).

A model's layers are cut into contiguous stages; each stage is a tensor/expert-parallel group of its own.  The hidden
state of a chunk travels stage to stage (rank i of a stage sends to rank i of the next: after the stage's last
all-reduce every rank holds the same rows, so no gather is needed), and the last stage returns the sampled token to
everyone.  Sends are asynchronous on the compute stream, so with chunked prefill stage s works on chunk c + 1 while
stage s + 1 works on chunk c; single-sequence decode is inherently serial across stages.

Reference behaviour: the ``layer_pp_4gpu`` policy (src/models/deepseek_v4/partition.py:241-270: contiguous layer
ranges per rank) and ``_forward_layer_pp`` (src/models/deepseek_v4/runtime.py:4850-4895: send/recv of the hidden
state, broadcast of the next token by the last stage).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


def split_layers(n_layers: int, n_stages: int, weights: list[float] | None = None) -> list[tuple[int, int]]:
    """Contiguous ``[lo, hi)`` layer ranges, balanced by ``weights`` (per-layer cost; default uniform).
    78 layers over 2 stages -> (0, 39), (39, 78)."""
    if n_stages < 1 or n_layers < n_stages:
        raise ValueError(f"cannot cut {n_layers} layers into {n_stages} stages")
    w = weights or [1.0] * n_layers
    if len(w) != n_layers:
        raise ValueError("one weight per layer")
    prefix = [0.0]
    for x in w:
        prefix.append(prefix[-1] + x)
    cuts = [0]
    for s in range(1, n_stages):
        target = prefix[-1] * s / n_stages
        lo_b, hi_b = cuts[-1] + 1, n_layers - (n_stages - s)
        cuts.append(min(range(lo_b, hi_b + 1), key=lambda b: (abs(prefix[b] - target), b)))
    cuts.append(n_layers)
    return [(cuts[i], cuts[i + 1]) for i in range(n_stages)]


@dataclass
class PipelineLayout:
    """Placement of a global rank in a ``stages x tp`` grid (stage-major: ranks [s*tp, (s+1)*tp) form stage s)."""
    rank: int
    world: int
    stages: int

    def __post_init__(self):
        if self.world % self.stages:
            raise ValueError("world size must be a multiple of the stage count")

    @property
    def tp(self) -> int:
        return self.world // self.stages

    @property
    def stage(self) -> int:
        return self.rank // self.tp

    @property
    def tp_rank(self) -> int:
        return self.rank % self.tp

    @property
    def is_first(self) -> bool:
        return self.stage == 0

    @property
    def is_last(self) -> bool:
        return self.stage == self.stages - 1

    @property
    def prev_rank(self) -> int | None:
        return None if self.is_first else self.rank - self.tp

    @property
    def next_rank(self) -> int | None:
        return None if self.is_last else self.rank + self.tp

    def stage_ranks(self, stage: int | None = None) -> list[int]:
        s = self.stage if stage is None else stage
        return list(range(s * self.tp, (s + 1) * self.tp))


class PipelineLink:
    """Transfers of one rank: hidden rows to/from the neighbouring stages and the token broadcast."""

    def __init__(self, layout: PipelineLayout, device, dtype=torch.bfloat16):
        self.layout, self.device, self.dtype = layout, torch.device(device), dtype
        self.bytes_sent = 0
        # every rank must create every group, in the same order
        self.stage_groups = [dist.new_group(layout.stage_ranks(s)) for s in range(layout.stages)] if layout.tp > 1 else None
        self._pending: list = []

    @property
    def stage_group(self):
        return None if self.stage_groups is None else self.stage_groups[self.layout.stage]

    def send_hidden(self, h: torch.Tensor) -> None:
        """Asynchronous on NCCL (ordered on the current stream); the tensor must stay alive until the next call."""
        nxt = self.layout.next_rank
        if nxt is None:
            return
        self._pending = [w for w in self._pending if not w[0].is_completed()]
        work = dist.isend(h.contiguous(), nxt)
        self._pending.append((work, h))
        self.bytes_sent += h.numel() * h.element_size()

    def recv_hidden(self, rows: int, hidden: int) -> torch.Tensor:
        prv = self.layout.prev_rank
        assert prv is not None
        h = torch.empty(rows, hidden, dtype=self.dtype, device=self.device)
        dist.recv(h, prv)
        return h

    def share_token(self, tok: torch.Tensor | None, n: int = 1) -> torch.Tensor:
        """The last stage's token ids (int32 [n]) to every rank.  Source: the first rank of the last stage."""
        src = self.layout.stage_ranks(self.layout.stages - 1)[0]
        if tok is None:
            tok = torch.zeros(n, dtype=torch.int32, device=self.device)
        tok = tok.to(self.device, torch.int32).contiguous()
        dist.broadcast(tok, src)
        return tok

    def drain(self) -> None:
        for w, _ in self._pending:
            w.wait()
        self._pending = []
