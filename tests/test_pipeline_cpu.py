"""Layer-pipeline host logic on CPU: layer cuts, rank grid, and the transfers over gloo ranks."""
import os
import subprocess
import sys

import pytest

from deepseek_v4_2080ti_b200.parallel import pp

HERE = os.path.dirname(os.path.abspath(__file__))


def test_split_layers():
    assert pp.split_layers(78, 2) == [(0, 39), (39, 78)]
    assert pp.split_layers(5, 5) == [(i, i + 1) for i in range(5)]
    cuts = pp.split_layers(43, 4)
    assert cuts[0][0] == 0 and cuts[-1][1] == 43 and all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
    assert max(hi - lo for lo, hi in cuts) - min(hi - lo for lo, hi in cuts) <= 1
    # a heavy layer pulls the cut towards itself
    assert pp.split_layers(10, 2, [1, 1, 1, 7, 1, 1, 1, 1, 1, 1]) == [(0, 4), (4, 10)]
    with pytest.raises(ValueError):
        pp.split_layers(3, 4)


def test_layout_grid():
    l = pp.PipelineLayout(5, 8, 2)
    assert (l.tp, l.stage, l.tp_rank, l.prev_rank, l.next_rank) == (4, 1, 1, 1, None)
    assert l.is_last and not l.is_first and l.stage_ranks() == [4, 5, 6, 7] and l.stage_ranks(0) == [0, 1, 2, 3]
    with pytest.raises(ValueError):
        pp.PipelineLayout(0, 6, 4)


@pytest.mark.parametrize("world,stages", [(2, 2), (4, 2), (3, 3)])
def test_pipeline_transfers_over_gloo(world, stages):
    env = dict(os.environ, PP_STAGES=str(stages), CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29800 + world + stages), os.path.join(HERE, "pp_cpu_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "PP_CPU_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-2000:])
