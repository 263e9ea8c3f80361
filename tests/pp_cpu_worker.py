"""CPU rank program (gloo) for the pipeline plumbing: hidden rows travel rank i -> rank i of the next stage, the token
comes back from the first rank of the last stage, stage groups reduce only inside a stage."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from deepseek_v4_2080ti_b200.parallel import pp, tp  # noqa: E402


def main() -> None:
    rank, world, _ = tp.init_distributed("gloo")
    stages = int(os.environ.get("PP_STAGES", "2"))
    layout = pp.PipelineLayout(rank, world, stages)
    link = pp.PipelineLink(layout, "cpu", dtype=torch.float32)
    for step in range(3):
        if layout.is_first:
            h = torch.full((5, 8), float(100 * step + layout.tp_rank))
        else:
            h = link.recv_hidden(5, 8)
            assert torch.all(h == 100 * step + layout.tp_rank + (layout.stage - 1)), (rank, step, h[0, 0])
            h = h + 1
        link.send_hidden(h)
        tok = torch.tensor([step * 7 + 3], dtype=torch.int32) if layout.is_last and layout.tp_rank == 0 else None
        got = link.share_token(tok)
        assert got.tolist() == [step * 7 + 3]
    link.drain()
    if layout.tp > 1:
        x = torch.tensor([float(rank)])
        dist.all_reduce(x, group=link.stage_group)
        assert x.item() == sum(layout.stage_ranks())
    if not layout.is_last:
        assert link.bytes_sent == 3 * 5 * 8 * 4
    dist.barrier()
    if rank == 0:
        print("PP_CPU_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
