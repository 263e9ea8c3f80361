"""Local tensor-parallel process group supervisor: one OS process per rank.

Behaviour kept from the reference (pocketllm/supervisor.py:55-626): per-rank environment
(RANK, LOCAL_RANK, WORLD_SIZE, TP_RANK, TP_WORLD, MASTER_ADDR, MASTER_PORT, POCKETLLM_NCCL_ID_PATH),
a private rendezvous directory, a parent-death signal so ranks never outlive the supervisor,
reader threads that watch stdout for the readiness marker, a start-up timeout, rank-death
monitoring, and SIGTERM -> SIGKILL escalation of whole process groups on shutdown.
There is no restart: one dead rank tears the group down.
"""
from __future__ import annotations

import collections
import ctypes
import os
import re
import shutil
import signal
import socket
import subprocess
import sys
import tempfile
import threading
import time
from dataclasses import dataclass, field
from typing import Sequence

from .api.errors import ConfigurationError, TensorParallelSupervisorError

READY_RE = re.compile(r"POCKETLLM_RANK_READY rank=(\d+)")
PR_SET_PDEATHSIG = 1


def _child_guard() -> None:
    """Runs in the child between fork and exec: die with the parent, own session."""
    try:
        libc = ctypes.CDLL(None, use_errno=True)
        libc.prctl(PR_SET_PDEATHSIG, signal.SIGKILL, 0, 0, 0)
    except Exception:
        pass
    if os.getppid() == 1:      # parent already gone
        os._exit(113)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@dataclass
class TensorParallelConfig:
    world_size: int
    command: Sequence[str]
    master_addr: str = "127.0.0.1"
    master_port: int = 0
    rendezvous_dir: str | None = None
    ready_timeout: float = 1800.0
    shutdown_grace: float = 10.0
    extra_env: dict[str, str] = field(default_factory=dict)
    ranks: list[int] | None = None           # which ranks to spawn (default: all)
    devices: list[int] | None = None         # rank -> CUDA device ordinal (default: rank)
    tail_lines: int = 40

    def __post_init__(self) -> None:
        if self.world_size < 1:
            raise ConfigurationError("world_size must be >= 1")
        if not self.command:
            raise ConfigurationError("command must not be empty")
        if self.ranks is None:
            self.ranks = list(range(self.world_size))
        if any(r < 0 or r >= self.world_size for r in self.ranks):
            raise ConfigurationError("ranks out of range")
        if self.devices is not None and len(self.devices) != self.world_size:
            raise ConfigurationError("devices must list one ordinal per rank")


class _Rank:
    def __init__(self, rank: int, proc: subprocess.Popen, tail: int):
        self.rank, self.proc = rank, proc
        self.ready = threading.Event()
        self.lines: collections.deque[str] = collections.deque(maxlen=tail)
        self.reader: threading.Thread | None = None


class TensorParallelSupervisor:
    def __init__(self, config: TensorParallelConfig, echo: bool = True):
        self.cfg = config
        self.echo = echo
        self._ranks: dict[int, _Rank] = {}
        self._own_dir = False
        self._dir: str | None = None
        self._stopping = False
        self._lock = threading.Lock()

    # ---- environment
    def _prepare_rendezvous(self) -> str:
        if self._dir:
            return self._dir
        if self.cfg.rendezvous_dir:
            os.makedirs(self.cfg.rendezvous_dir, exist_ok=True)
            self._dir = self.cfg.rendezvous_dir
        else:
            self._dir = tempfile.mkdtemp(prefix="pocketllm-tp-")
            self._own_dir = True
        if not self.cfg.master_port:
            self.cfg.master_port = _free_port()
        stale = os.path.join(self._dir, "nccl_id")
        for p in (stale, stale + ".cmdsock"):
            if os.path.exists(p):
                os.unlink(p)
        return self._dir

    def rank_env(self, rank: int) -> dict[str, str]:
        d = self._prepare_rendezvous()
        dev = self.cfg.devices[rank] if self.cfg.devices else rank
        env = {"RANK": str(rank), "LOCAL_RANK": str(dev), "WORLD_SIZE": str(self.cfg.world_size),
               "TP_RANK": str(rank), "TP_WORLD": str(self.cfg.world_size), "MASTER_ADDR": self.cfg.master_addr,
               "MASTER_PORT": str(self.cfg.master_port), "POCKETLLM_NCCL_ID_PATH": os.path.join(d, "nccl_id"),
               "POCKETLLM_RENDEZVOUS_DIR": d}
        env.update(self.cfg.extra_env)
        return env

    # ---- spawn
    def _read(self, r: _Rank) -> None:
        assert r.proc.stdout is not None
        for raw in r.proc.stdout:
            line = raw.rstrip("\n")
            r.lines.append(line)
            m = READY_RE.search(line)
            if m and int(m.group(1)) == r.rank:
                r.ready.set()
            elif self.echo:
                print(f"[rank {r.rank}] {line}", file=sys.stderr, flush=True)

    def _spawn(self, rank: int) -> None:
        env = dict(os.environ)
        env.update(self.rank_env(rank))
        proc = subprocess.Popen(list(self.cfg.command), env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                text=True, bufsize=1, start_new_session=True, preexec_fn=_child_guard)
        r = _Rank(rank, proc, self.cfg.tail_lines)
        r.reader = threading.Thread(target=self._read, args=(r,), daemon=True, name=f"tp-rank-{rank}-reader")
        r.reader.start()
        self._ranks[rank] = r

    def start(self) -> None:
        with self._lock:
            if self._ranks:
                return
            try:
                for rank in self.cfg.ranks or []:
                    self._spawn(rank)
            except Exception:
                self._shutdown_children()
                raise

    def _tail(self, r: _Rank) -> str:
        return "\n".join(r.lines) or "<no output>"

    def wait_ready(self, timeout: float | None = None) -> None:
        deadline = time.monotonic() + (self.cfg.ready_timeout if timeout is None else timeout)
        pending = dict(self._ranks)
        while pending:
            for rank, r in list(pending.items()):
                if r.ready.is_set():
                    del pending[rank]
                    continue
                code = r.proc.poll()
                if code is not None:
                    if r.reader:
                        r.reader.join(timeout=1.0)
                    if r.ready.is_set():
                        del pending[rank]
                        continue
                    self._shutdown_children()
                    raise TensorParallelSupervisorError(
                        f"rank {rank} exited with code {code} before becoming ready; last output:\n{self._tail(r)}")
            if pending and time.monotonic() > deadline:
                waiting = sorted(pending)
                self._shutdown_children()
                raise TensorParallelSupervisorError(f"ranks {waiting} were not ready within the timeout")
            if pending:
                time.sleep(0.02)

    def poll(self) -> tuple[int, int] | None:
        """(rank, exit code) of the first rank found dead, else None."""
        for rank, r in self._ranks.items():
            code = r.proc.poll()
            if code is not None:
                return rank, code
        return None

    # ---- shutdown
    def _signal_group(self, r: _Rank, sig: int) -> None:
        try:
            os.killpg(r.proc.pid, sig)
        except (ProcessLookupError, PermissionError):
            try:
                r.proc.send_signal(sig)
            except ProcessLookupError:
                pass

    def _shutdown_children(self) -> None:
        self._stopping = True
        live = [r for r in self._ranks.values() if r.proc.poll() is None]
        for r in live:
            self._signal_group(r, signal.SIGTERM)
        deadline = time.monotonic() + self.cfg.shutdown_grace
        while live and time.monotonic() < deadline:
            live = [r for r in live if r.proc.poll() is None]
            if live:
                time.sleep(0.02)
        for r in live:
            self._signal_group(r, signal.SIGKILL)
        for r in self._ranks.values():
            try:
                r.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                pass

    def cleanup(self) -> None:
        self._shutdown_children()
        if self._own_dir and self._dir and os.path.isdir(self._dir):
            shutil.rmtree(self._dir, ignore_errors=True)
        self._ranks.clear()

    def run(self) -> int:
        """Start, wait for readiness, then babysit until a rank exits or a signal arrives. Returns an exit code."""
        caught: list[int] = []
        old = {}
        if threading.current_thread() is threading.main_thread():
            for s in (signal.SIGINT, signal.SIGTERM):
                old[s] = signal.signal(s, lambda n, f: caught.append(n))
        try:
            self.start()
            self.wait_ready()
            while not caught:
                dead = self.poll()
                if dead is not None:
                    rank, code = dead
                    r = self._ranks[rank]
                    if code != 0:
                        raise TensorParallelSupervisorError(
                            f"rank {rank} died with exit code {code}; last output:\n{self._tail(r)}")
                    return 0
                time.sleep(0.1)
            return 128 + caught[0]
        finally:
            self.cleanup()
            for s, h in old.items():
                signal.signal(s, h)
