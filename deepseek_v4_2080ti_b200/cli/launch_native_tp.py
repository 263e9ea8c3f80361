"""Start the native executable tensor-parallel: one process per GPU of this machine, a fresh rendezvous file, rank 0 on
this terminal.

    python -m deepseek_v4_2080ti_b200.cli.launch_native_tp --tp 4 -- --ckpt DIR --qwen-persistent-stdin --max-context 9000

Every rank gets ``--tp-world N --tp-rank R --device R --nccl-id-path FILE`` appended to the arguments after ``--``.
Rank 0 inherits stdin / stdout (so the stdin modes and ``--serve`` work as with one process); the other ranks' output
goes to ``<log-dir>/rank<R>.log``.  If any rank exits, the others are terminated (SIGTERM, then SIGKILL after a grace
period), and the launcher returns the first non-zero exit code.  Counterpart of the reference's per-rank launch scripts
(scripts/run_cpp_serve_tp4.sh: four processes, one visible device each, a file rendezvous).
"""
from __future__ import annotations

import argparse
import os
import signal
import subprocess
import sys
import tempfile
import time


def default_executable() -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "pocketllm_engine")


def launch(tp: int, engine_args: list[str], exe: str | None = None, log_dir: str | None = None, grace: float = 10.0,
           devices: list[int] | None = None) -> int:
    if tp < 1:
        raise ValueError("--tp must be >= 1")
    devices = devices or list(range(tp))
    if len(devices) != tp:
        raise ValueError("--devices must name one device per rank")
    exe = exe or default_executable()
    work = log_dir or tempfile.mkdtemp(prefix="pocketllm-tp-")
    os.makedirs(work, exist_ok=True)
    id_path = os.path.join(work, f"nccl_id_{os.getpid()}")
    procs: list[subprocess.Popen] = []
    logs = []
    try:
        for r in range(tp):
            cmd = [exe, *engine_args, "--tp-world", str(tp), "--tp-rank", str(r), "--device", str(devices[r]), "--nccl-id-path", id_path]
            if r == 0:
                procs.append(subprocess.Popen(cmd))
            else:
                f = open(os.path.join(work, f"rank{r}.log"), "wb")
                logs.append(f)
                procs.append(subprocess.Popen(cmd, stdin=subprocess.DEVNULL, stdout=f, stderr=subprocess.STDOUT))
        code = 0
        while True:
            done = [(r, p.poll()) for r, p in enumerate(procs)]
            exited = [(r, c) for r, c in done if c is not None]
            if exited:
                code = next((c for _, c in exited if c != 0), 0)
                if len(exited) == tp or code != 0 or any(r == 0 for r, _ in exited):
                    break
            time.sleep(0.05)
        # whoever is still running has lost its group
        deadline = time.time() + grace
        for p in procs:
            if p.poll() is None:
                p.send_signal(signal.SIGTERM)
        for p in procs:
            while p.poll() is None and time.time() < deadline:
                time.sleep(0.05)
            if p.poll() is None:
                p.kill()
                p.wait()
        if code == 0:
            code = next((p.returncode for p in procs if p.returncode not in (0, -signal.SIGTERM)), 0)
        if code != 0:
            for r in range(1, tp):
                path = os.path.join(work, f"rank{r}.log")
                if os.path.exists(path) and os.path.getsize(path):
                    tail = open(path, "rb").read()[-600:].decode(errors="replace")
                    sys.stderr.write(f"--- rank {r} ({path}) ---\n{tail}\n")
        return code if code >= 0 else 128 - code
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        for f in logs:
            f.close()
        try:
            os.remove(id_path)
        except OSError:
            pass


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    rest: list[str] = []
    if "--" in argv:
        i = argv.index("--")
        argv, rest = argv[:i], argv[i + 1:]
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--tp", type=int, required=True)
    ap.add_argument("--exe", default=None)
    ap.add_argument("--log-dir", default=None)
    ap.add_argument("--devices", default="", help="comma-separated device indices, one per rank (default 0..tp-1)")
    ap.add_argument("--grace", type=float, default=10.0)
    a = ap.parse_args(argv)
    if not rest:
        ap.error("give the engine's arguments after --")
    for flag in ("--tp-world", "--tp-rank", "--nccl-id-path", "--device"):
        if flag in rest:
            ap.error(f"{flag} is set by the launcher")
    devs = [int(x) for x in a.devices.split(",") if x] or None
    return launch(a.tp, rest, a.exe, a.log_dir, a.grace, devs)


if __name__ == "__main__":
    sys.exit(main())
