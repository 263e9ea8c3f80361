"""Rank program of the pipeline tests (launched by torch.distributed.run): a 2-stage layer pipeline of the MLA + MoE
runtime with GGUF weights must generate the tokens of the unsplit model.  Prints ``PP_WORKER_OK``."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from deepseek_v4_2080ti_b200.models import mla_moe as mm  # noqa: E402
from deepseek_v4_2080ti_b200.models import mla_moe_gpu as mg  # noqa: E402
from deepseek_v4_2080ti_b200.ops import _lib  # noqa: E402
from deepseek_v4_2080ti_b200.parallel import pp, tp  # noqa: E402


def main() -> None:
    rank, world, local = tp.init_distributed()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    stages = 2
    layout = pp.PipelineLayout(rank, world, stages)
    link = pp.PipelineLink(layout, dev)
    cfg = mm.MlaMoeConfig(vocab_size=512, hidden_size=256, num_layers=4, first_dense_layers=1, dense_intermediate=256,
                          q_lora_rank=256, kv_lora_rank=128, num_heads=4 * layout.tp, qk_nope_dim=64, qk_rope_dim=32,
                          v_head_dim=128, index_heads=4, index_dim=32, index_topk=24, num_experts=8, experts_per_token=2,
                          num_shared_experts=1, expert_intermediate=256, score_func="sigmoid", route_scale=2.5,
                          expert_format="bf16")
    state = list(mm.synth_state(cfg, seed=6, std=0.05))
    prompt = torch.randint(0, cfg.vocab_size, (90,), generator=torch.Generator().manual_seed(5))
    mix = mg.GLM_GGUF_MIX
    whole = mg.MlaMoeGpuRuntime(cfg, mg.MlaMoeGpuWeights(cfg, iter(state), dev, gguf_mix=mix), max_context=256)
    want, _ = whole.generate(prompt, 8, chunk=32)
    del whole
    lo, hi = pp.split_layers(cfg.num_layers, stages)[layout.stage]
    comm = None
    if layout.tp > 1:
        comm = tp.TPComm(group=link.stage_group)
    w = mg.MlaMoeGpuWeights(cfg, iter(state), dev, rank=layout.tp_rank, world=layout.tp, layer_range=(lo, hi), gguf_mix=mix)
    assert (w.embed is not None) == layout.is_first and (w.head is not None) == layout.is_last
    rt = mg.MlaMoeGpuRuntime(cfg, w, max_context=256, comm=comm, pipeline=link)
    got, _ = rt.generate(prompt, 8, chunk=32)
    torch.cuda.synchronize()
    _lib.check_status()
    assert got[:4] == want[:4], (rank, got, want)
    ref = torch.tensor(got, device=dev)
    dist.broadcast(ref, 0)
    assert ref.tolist() == got, "stages disagree on the token stream"
    if not layout.is_last:
        assert link.bytes_sent == (90 + 7) * cfg.hidden_size * 2
    dist.barrier()
    if rank == 0:
        print("PP_WORKER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
