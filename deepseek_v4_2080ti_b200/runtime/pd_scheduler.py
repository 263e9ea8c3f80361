"""Prefill / decode phase scheduling with per-phase host resources.

Requests wait in a prefill queue, move to a decode queue once their prompt is in the cache, and decode always goes
first.  Entering a phase applies that phase's host settings: CPU affinity, worker-thread count of the host expert
kernels, and (optionally) pausing an external expert-server process while the GPUs prefill.  Settings come from a
``PhaseResources`` object per phase instead of process-wide environment switches.

Reference behaviour: PDScheduler / PDExecutionFacade (src/runtime/pd_scheduler.py:53-263): decode-first queues, per-phase
affinity / thread / NUMA policy, SIGSTOP / SIGCONT of the CPU expert server between phases."""
from __future__ import annotations

import collections
import os
import signal
from dataclasses import dataclass, field
from typing import Any, Callable, Deque, Iterator

PHASES = ("prefill", "decode")


@dataclass
class PhaseResources:
    cpus: tuple[int, ...] = ()             # CPU affinity of this process during the phase (empty = unchanged)
    host_threads: int = 0                  # worker threads of the host expert kernels (0 = unchanged)
    pause_server: bool = False             # stop the external expert server while this phase runs


@dataclass
class PDRequest:
    request_id: int
    prompt_tokens: list[int]
    max_new_tokens: int
    phase: str = "prefill"
    kv_owned: bool = False
    output: list[int] = field(default_factory=list)


def parse_cpu_list(spec: str) -> tuple[int, ...]:
    """``"0-3,8,10-11"`` -> (0, 1, 2, 3, 8, 10, 11)."""
    out: list[int] = []
    for part in spec.split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            lo, hi = part.split("-", 1)
            out.extend(range(int(lo), int(hi) + 1))
        else:
            out.append(int(part))
    return tuple(sorted(set(out)))


class PDScheduler:
    def __init__(self, resources: dict[str, PhaseResources] | None = None, server_pid: int | None = None,
                 set_host_threads: Callable[[int], None] | None = None, set_affinity: Callable[[set[int]], None] | None = None,
                 send_signal: Callable[[int, int], None] | None = None):
        self.prefill_queue: Deque[PDRequest] = collections.deque()
        self.decode_queue: Deque[PDRequest] = collections.deque()
        self.resources = {p: (resources or {}).get(p, PhaseResources()) for p in PHASES}
        self.server_pid = server_pid
        self._set_threads = set_host_threads
        self._set_affinity = set_affinity or (lambda cpus: os.sched_setaffinity(0, cpus) if hasattr(os, "sched_setaffinity") else None)
        self._signal = send_signal or os.kill
        self._next_id = 0
        self.phase: str | None = None
        self.server_paused = False
        self.phase_switches = 0

    # ---- queues
    def submit(self, prompt_tokens: list[int], max_new_tokens: int) -> PDRequest:
        r = PDRequest(self._next_id, list(prompt_tokens), int(max_new_tokens))
        self._next_id += 1
        self.prefill_queue.append(r)
        return r

    def has_work(self) -> bool:
        return bool(self.decode_queue) or bool(self.prefill_queue)

    def next_step(self) -> tuple[PDRequest, str] | None:
        if self.decode_queue:
            return self.decode_queue[0], "decode"
        if self.prefill_queue:
            return self.prefill_queue[0], "prefill"
        return None

    def mark_prefill_done(self, r: PDRequest) -> None:
        if r in self.prefill_queue:
            self.prefill_queue.remove(r)
        r.phase, r.kv_owned = "decode", True
        self.decode_queue.append(r)

    def mark_request_done(self, r: PDRequest) -> None:
        for q in (self.decode_queue, self.prefill_queue):
            if r in q:
                q.remove(r)
        r.kv_owned = False
        r.phase = "done"

    # ---- per-phase host resources
    def apply_phase(self, phase: str) -> None:
        if phase not in PHASES:
            raise ValueError(f"unknown phase {phase!r}")
        if self.phase == phase:
            return
        self.phase = phase
        self.phase_switches += 1
        res = self.resources[phase]
        if res.cpus:
            try:
                self._set_affinity(set(res.cpus))
            except OSError:
                pass
        if res.host_threads > 0 and self._set_threads is not None:
            self._set_threads(res.host_threads)
        self._pause_server(res.pause_server)

    def _pause_server(self, paused: bool) -> None:
        if self.server_pid is None or paused == self.server_paused:
            return
        try:
            self._signal(self.server_pid, signal.SIGSTOP if paused else signal.SIGCONT)
            self.server_paused = paused
        except ProcessLookupError:
            self.server_pid = None
        except OSError:
            pass

    # ---- driving loop
    def run(self, prefill_fn: Callable[[PDRequest], int], decode_fn: Callable[[PDRequest], int],
            is_eos: Callable[[int], bool] = lambda t: False) -> Iterator[PDRequest]:
        """Drain the queues: ``prefill_fn(request) -> first token``, ``decode_fn(request) -> next token`` (both see
        ``request.output``).  Yields every request as it completes."""
        while self.has_work():
            r, phase = self.next_step()
            self.apply_phase(phase)
            tok = prefill_fn(r) if phase == "prefill" else decode_fn(r)
            r.output.append(tok)
            if phase == "prefill":
                self.mark_prefill_done(r)
            if is_eos(tok) or len(r.output) >= r.max_new_tokens:
                self.mark_request_done(r)
                yield r
        self._pause_server(False)
