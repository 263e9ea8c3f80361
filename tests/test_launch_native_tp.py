"""The per-GPU launcher of the native executable, against a stand-in executable: argument fan-out, rank 0 on the
terminal, logs of the other ranks, and group teardown when a rank dies."""
import os
import stat
import subprocess
import sys
import textwrap
import time

from deepseek_v4_2080ti_b200.cli import launch_native_tp as lt


def _fake(tmp_path, body):
    p = tmp_path / "fake_engine"
    p.write_text("#!" + sys.executable + "\n" + textwrap.dedent(body))
    p.chmod(p.stat().st_mode | stat.S_IEXEC)
    return str(p)


def test_ranks_get_their_arguments_and_rank0_keeps_the_terminal(tmp_path):
    exe = _fake(tmp_path, """
        import sys, os, time
        a = sys.argv[1:]
        rank = a[a.index("--tp-rank") + 1]
        print("rank", rank, "world", a[a.index("--tp-world") + 1], "device", a[a.index("--device") + 1],
              "id", os.path.basename(a[a.index("--nccl-id-path") + 1]), "extra", a[0], a[1], flush=True)
        if rank == "0":
            print("echo", sys.stdin.readline().strip(), flush=True)
        else:
            time.sleep(0.3)
    """)
    r = subprocess.run([sys.executable, "-m", "deepseek_v4_2080ti_b200.cli.launch_native_tp", "--tp", "3", "--exe", exe,
                        "--log-dir", str(tmp_path / "logs"), "--devices", "4,5,6", "--", "--ckpt", "DIR"],
                       input="hello\n", capture_output=True, text=True, timeout=60,
                       env=dict(os.environ, PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    assert r.returncode == 0, r.stderr
    assert "rank 0 world 3 device 4" in r.stdout and "echo hello" in r.stdout and "extra --ckpt DIR" in r.stdout
    for rank, dev in ((1, 5), (2, 6)):
        log = (tmp_path / "logs" / f"rank{rank}.log").read_text()
        assert f"rank {rank} world 3 device {dev}" in log
    assert not [f for f in os.listdir(tmp_path / "logs") if f.startswith("nccl_id_")]        # the rendezvous file is removed


def test_a_dying_rank_takes_the_group_down_and_its_log_is_shown(tmp_path, capsys):
    exe = _fake(tmp_path, """
        import sys, time
        a = sys.argv[1:]
        if a[a.index("--tp-rank") + 1] == "1":
            print("rank 1 cannot load its shard", flush=True)
            sys.exit(7)
        time.sleep(60)
    """)
    t0 = time.time()
    code = lt.launch(2, ["--ckpt", "DIR"], exe, str(tmp_path / "logs"), grace=5.0)
    assert code == 7 and time.time() - t0 < 20
    assert "rank 1 cannot load its shard" in capsys.readouterr().err


def test_launcher_owns_the_rank_arguments(tmp_path):
    import pytest
    with pytest.raises(SystemExit):
        lt.main(["--tp", "2", "--", "--ckpt", "D", "--tp-rank", "1"])
    with pytest.raises(SystemExit):
        lt.main(["--tp", "2"])
    with pytest.raises(ValueError):
        lt.launch(2, ["--ckpt", "D"], "/bin/true", str(tmp_path), devices=[0])
