"""Dependency-free Prometheus text registry: counters, gauges and summaries with p50/p90/p99
(reference surface: pocketllm/server/metrics.py:12-72)."""
from __future__ import annotations

import threading
from collections import defaultdict, deque


def _labels(labels: dict[str, str] | None) -> str:
    if not labels:
        return ""
    inner = ",".join(f'{k}="{str(v).replace(chr(92), chr(92) * 2).replace(chr(34), chr(92) + chr(34))}"' for k, v in sorted(labels.items()))
    return "{" + inner + "}"


class Metrics:
    def __init__(self, window: int = 2048, prefix: str = "pocketllm_"):
        self._lock = threading.Lock()
        self._prefix = prefix
        self._counters: dict[tuple[str, str], float] = defaultdict(float)
        self._gauges: dict[tuple[str, str], float] = {}
        self._samples: dict[tuple[str, str], deque] = defaultdict(lambda: deque(maxlen=window))
        self._sums: dict[tuple[str, str], list[float]] = defaultdict(lambda: [0.0, 0.0])
        self._help: dict[str, str] = {}

    def describe(self, name: str, text: str) -> None:
        self._help[name] = text

    def inc(self, name: str, value: float = 1.0, labels: dict[str, str] | None = None) -> None:
        with self._lock:
            self._counters[(name, _labels(labels))] += value

    def set(self, name: str, value: float, labels: dict[str, str] | None = None) -> None:
        with self._lock:
            self._gauges[(name, _labels(labels))] = float(value)

    def add(self, name: str, delta: float, labels: dict[str, str] | None = None) -> None:
        with self._lock:
            key = (name, _labels(labels))
            self._gauges[key] = self._gauges.get(key, 0.0) + delta

    def observe(self, name: str, value: float, labels: dict[str, str] | None = None) -> None:
        with self._lock:
            key = (name, _labels(labels))
            self._samples[key].append(float(value))
            s = self._sums[key]
            s[0] += float(value)
            s[1] += 1

    @staticmethod
    def _quantile(sorted_vals: list[float], q: float) -> float:
        if not sorted_vals:
            return 0.0
        pos = q * (len(sorted_vals) - 1)
        lo = int(pos)
        hi = min(lo + 1, len(sorted_vals) - 1)
        return sorted_vals[lo] + (sorted_vals[hi] - sorted_vals[lo]) * (pos - lo)

    def render(self) -> str:
        out: list[str] = []
        with self._lock:
            seen: set[str] = set()

            def header(name: str, kind: str) -> None:
                if name not in seen:
                    seen.add(name)
                    if name in self._help:
                        out.append(f"# HELP {self._prefix}{name} {self._help[name]}")
                    out.append(f"# TYPE {self._prefix}{name} {kind}")

            for (name, lab), v in sorted(self._counters.items()):
                header(name, "counter")
                out.append(f"{self._prefix}{name}{lab} {v:g}")
            for (name, lab), v in sorted(self._gauges.items()):
                header(name, "gauge")
                out.append(f"{self._prefix}{name}{lab} {v:g}")
            for (name, lab), dq in sorted(self._samples.items()):
                header(name, "summary")
                vals = sorted(dq)
                base = lab[1:-1] if lab else ""
                for q in (0.5, 0.9, 0.99):
                    ql = "{" + (base + "," if base else "") + f'quantile="{q}"' + "}"
                    out.append(f"{self._prefix}{name}{ql} {self._quantile(vals, q):g}")
                s = self._sums[(name, lab)]
                out.append(f"{self._prefix}{name}_sum{lab} {s[0]:g}")
                out.append(f"{self._prefix}{name}_count{lab} {s[1]:g}")
        return "\n".join(out) + "\n"
