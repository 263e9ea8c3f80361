"""Page-cache warming for large checkpoints: advise the kernel (POSIX_FADV_WILLNEED / SEQUENTIAL) and stream the files
through a few reader threads, so the first mmap access of each tensor does not stall on disk.

Reference behaviour: src/loader/gguf/prewarm.py:28-140."""
from __future__ import annotations

import os
import threading
import time
from typing import Iterable, Sequence


def _fadvise(fd: int) -> None:
    adv = getattr(os, "posix_fadvise", None)
    if adv is None:
        return
    for flag in ("POSIX_FADV_SEQUENTIAL", "POSIX_FADV_WILLNEED"):
        try:
            adv(fd, 0, 0, getattr(os, flag))
        except (OSError, AttributeError):
            pass


def prewarm_paths(paths: Sequence[str], threads: int = 4, chunk_bytes: int = 8 << 20, max_bytes: int | None = None,
                  ranges: Iterable[tuple[str, int, int]] | None = None) -> dict:
    """Read every file (or only the ``(path, offset, nbytes)`` ranges: e.g. this rank's experts) once.
    Returns ``{"files", "bytes", "seconds"}``."""
    work: list[tuple[str, int, int]] = list(ranges) if ranges is not None else [(p, 0, os.path.getsize(p)) for p in paths]
    lock = threading.Lock()
    state = {"next": 0, "bytes": 0}
    budget = max_bytes

    def run() -> None:
        while True:
            with lock:
                i = state["next"]
                state["next"] += 1
            if i >= len(work):
                return
            path, off, n = work[i]
            fd = os.open(path, os.O_RDONLY)
            try:
                _fadvise(fd)
                done = 0
                while done < n:
                    with lock:
                        if budget is not None and state["bytes"] >= budget:
                            return
                    got = len(os.pread(fd, min(chunk_bytes, n - done), off + done))
                    if got == 0:
                        break
                    done += got
                    with lock:
                        state["bytes"] += got
            finally:
                os.close(fd)

    t0 = time.time()
    ts = [threading.Thread(target=run, daemon=True) for _ in range(max(1, min(threads, len(work))))]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    return {"files": len({w[0] for w in work}), "bytes": state["bytes"], "seconds": time.time() - t0}


def prewarm_bundle(bundle, names: Iterable[str] | None = None, threads: int = 4, max_bytes: int | None = None) -> dict:
    """Warm the byte ranges of the named tensors of a ``GGUFBundle`` (all tensors when ``names`` is None)."""
    ranges = []
    for name, ti in bundle.tensors.items():
        if names is not None and name not in names:
            continue
        ranges.append((ti.file.path, ti.file.data_start + ti.offset, ti.nbytes))
    return prewarm_paths([], threads=threads, max_bytes=max_bytes, ranges=ranges)
