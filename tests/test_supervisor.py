"""Tensor-parallel supervisor with tiny CPU child scripts: ready, early exit, hang, ignored SIGTERM, orphan guard."""
import os
import signal
import subprocess
import sys
import time

import pytest

from pocketllm import TensorParallelSupervisorError
from pocketllm.supervisor import TensorParallelConfig, TensorParallelSupervisor

READY = "import os,sys,time; print('POCKETLLM_RANK_READY rank=' + os.environ['RANK'], flush=True); "


def sup(script, world=2, **kw):
    return TensorParallelSupervisor(TensorParallelConfig(world_size=world, command=[sys.executable, "-c", script], **kw), echo=False)


def test_ready_env_and_clean_shutdown(tmp_path):
    out = tmp_path / "env"
    script = READY + f"open(r'{out}' + os.environ['RANK'], 'w').write(os.environ['WORLD_SIZE'] + ' ' + os.environ['TP_RANK'] + ' ' + os.environ['MASTER_ADDR'] + ' ' + os.environ['POCKETLLM_NCCL_ID_PATH']); time.sleep(60)"
    s = sup(script, world=3)
    s.start()
    s.wait_ready(timeout=20)
    assert s.poll() is None
    s.cleanup()
    for r in range(3):
        w, tr, addr, path = open(str(out) + str(r)).read().split()
        assert (w, tr, addr) == ("3", str(r), "127.0.0.1") and path.endswith("nccl_id")
    assert not os.path.exists(os.path.dirname(path))      # private rendezvous dir removed


def test_early_exit_reports_output_tail():
    s = sup("import sys; print('boom detail'); sys.exit(7)")
    s.start()
    with pytest.raises(TensorParallelSupervisorError) as e:
        s.wait_ready(timeout=20)
    assert "code 7" in str(e.value) and "boom detail" in str(e.value)


def test_ready_timeout_kills_hung_ranks():
    s = sup("import time; time.sleep(60)")
    s.start()
    t0 = time.time()
    with pytest.raises(TensorParallelSupervisorError):
        s.wait_ready(timeout=0.5)
    assert time.time() - t0 < 15 and all(r.proc.poll() is not None for r in s._ranks.values())


def test_sigterm_ignored_escalates_to_sigkill():
    script = "import signal,time,os; signal.signal(signal.SIGTERM, signal.SIG_IGN); print('POCKETLLM_RANK_READY rank=' + os.environ['RANK'], flush=True); time.sleep(60)"
    s = sup(script, world=1, shutdown_grace=0.5)
    s.start()
    s.wait_ready(timeout=20)
    proc = s._ranks[0].proc
    s.cleanup()
    assert proc.poll() == -signal.SIGKILL


def test_run_returns_error_when_a_rank_dies():
    script = READY + "time.sleep(0.3 if os.environ['RANK']=='1' else 60); sys.exit(3 if os.environ['RANK']=='1' else 0)"
    with pytest.raises(TensorParallelSupervisorError) as e:
        sup(script).run()
    assert "rank 1" in str(e.value)


def test_ranks_die_with_the_supervisor(tmp_path):
    """SIGKILL the supervising process: the parent-death signal must take the ranks down with it."""
    pidfile = tmp_path / "pids"
    child = READY + f"open(r'{pidfile}', 'a').write(str(os.getpid()) + '\\n'); time.sleep(120)"
    parent = (f"import sys; sys.path.insert(0, r'{os.getcwd()}')\n"
              "from pocketllm.supervisor import TensorParallelConfig, TensorParallelSupervisor\n"
              f"s = TensorParallelSupervisor(TensorParallelConfig(world_size=2, command=[sys.executable, '-c', {child!r}]), echo=False)\n"
              "s.start(); s.wait_ready(timeout=20); print('UP', flush=True)\n"
              "import time; time.sleep(120)\n")
    p = subprocess.Popen([sys.executable, "-c", parent], stdout=subprocess.PIPE, text=True)
    assert p.stdout.readline().strip() == "UP"
    pids = [int(x) for x in open(pidfile).read().split()]
    p.kill()
    p.wait()
    deadline = time.time() + 10
    alive = pids
    while alive and time.time() < deadline:
        alive = [q for q in alive if os.path.exists(f"/proc/{q}") and "Z" not in open(f"/proc/{q}/stat").read().split()[2]]
        time.sleep(0.1)
    assert not alive


def test_config_validation():
    from pocketllm import ConfigurationError
    with pytest.raises(ConfigurationError):
        TensorParallelConfig(world_size=0, command=["x"])
    with pytest.raises(ConfigurationError):
        TensorParallelConfig(world_size=2, command=[])
    with pytest.raises(ConfigurationError):
        TensorParallelConfig(world_size=2, command=["x"], devices=[0])
