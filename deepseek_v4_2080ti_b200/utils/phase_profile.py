"""Per-site phase profiling of a forward pass: NVTX ranges and device-timed accumulators.

Modes:  ``off`` (the default: a scope costs one attribute test), ``range`` (NVTX range push/pop only: no
synchronisation, the pipeline is unchanged, ranges show up in a timeline capture), ``timed`` (a CUDA-event pair per
scope, recorded on the launching stream; elapsed times are read only in ``report()``, after one synchronise, so the hot
path never waits).  Sites are named like the reference's (``"lin.qkv"``, ``"ar.mlp"``, ``"full.attn_kernel"``...).

Reference behaviour: PhaseScope / QwenRuntimeTelemetry (cpp_engine/engine/qwen_engine.cpp:1829-1897: NVTX range, or
synchronise both ends and accumulate wall time per named site), GLM_PROFILE section timers
(src/models/glm_dsa/architecture.py:32-118), Qwen4Exp Profiler scopes (src/models/qwen4_exp/profiler.py:22-120)."""
from __future__ import annotations

import contextlib
from collections import defaultdict

import torch


class PhaseProfiler:
    def __init__(self, mode: str = "off"):
        self.set_mode(mode)
        self._events: dict[str, list] = defaultdict(list)
        self._calls: dict[str, int] = defaultdict(int)

    def set_mode(self, mode: str) -> None:
        if mode not in ("off", "range", "timed"):
            raise ValueError(f"unknown profile mode {mode!r}")
        self.mode = mode
        self.enabled = mode != "off"

    @contextlib.contextmanager
    def _scope(self, name: str):
        cuda = torch.cuda.is_available()
        if self.mode == "range":
            if cuda:
                torch.cuda.nvtx.range_push(name)
            try:
                yield
            finally:
                if cuda:
                    torch.cuda.nvtx.range_pop()
            return
        self._calls[name] += 1
        if not cuda:
            import time
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self._events[name].append(("host", (time.perf_counter() - t0) * 1e3))
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        try:
            yield
        finally:
            b.record()
            self._events[name].append((a, b))

    _NULL = contextlib.nullcontext()

    def scope(self, name: str):
        return self._scope(name) if self.enabled else self._NULL

    def reset(self) -> None:
        self._events.clear()
        self._calls.clear()

    def report(self) -> dict[str, dict[str, float]]:
        """site -> {"calls", "ms", "share"}; synchronises once."""
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        out = {}
        for name, evs in self._events.items():
            ms = sum(e[1] if e[0] == "host" else e[0].elapsed_time(e[1]) for e in evs)
            out[name] = {"calls": self._calls[name], "ms": ms}
        total = sum(v["ms"] for v in out.values()) or 1.0
        for v in out.values():
            v["share"] = v["ms"] / total
        return dict(sorted(out.items(), key=lambda kv: -kv[1]["ms"]))

    def format(self) -> str:
        return "\n".join(f"phase site={n} calls={v['calls']} ms={v['ms']:.3f} share={v['share']:.3f}" for n, v in self.report().items())


PROFILER = PhaseProfiler()        # process-wide instance the runtimes consult
