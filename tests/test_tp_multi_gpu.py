"""Multi-GPU tensor parallelism: peer-memory collectives and the fused GEMM + all-reduce against NCCL, and a
tensor-parallel model against the single-rank model.  One process per GPU over NCCL/NVLink; skipped with < 2 GPUs."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_worker(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + world), os.path.join(HERE, "tp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0 and "TP_WORKER_OK" in r.stdout, (r.stdout[-3000:], r.stderr[-8000:])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("world", [2, 4])
def test_pipeline_worker(world):
    """2-stage layer pipeline (1 or 2 tensor-parallel ranks per stage) == the unsplit model."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29700 + world), os.path.join(HERE, "pp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0 and "PP_WORKER_OK" in r.stdout, (r.stdout[-3000:], r.stderr[-8000:])
