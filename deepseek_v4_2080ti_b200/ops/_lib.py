"""ctypes loader for the sm_100a kernel library (``lib/libb200_kernels.so``).

The library exports plain C launchers (see ``csrc/kernels/ops.h``); Python passes
``tensor.data_ptr()`` and the current CUDA stream handle.  There is deliberately
no PyTorch fallback: on a machine with a GPU a missing library is an error, so a
silently slower eager path can never stand in for the kernels.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent.parent
_LIB_PATH = _PKG / "lib" / "libb200_kernels.so"
_lib = None
_status: dict[int, torch.Tensor] = {}

ERR_NAMES = {
    1: "TMA completion wait expired",
    2: "pipeline stage wait expired",
    3: "accumulator wait expired",
    4: "peer flag wait expired",
    5: "weight-decode wait expired",
    6: "bad argument",
}


class KernelError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            if os.environ.get("B200_AUTOBUILD", "1") == "1":
                from .. import build as _build

                _build.build_kernels()
            if not _LIB_PATH.exists():
                raise KernelError(f"kernel library not built: {_LIB_PATH} (run python -m deepseek_v4_2080ti_b200.build)")
        _lib = ctypes.CDLL(str(_LIB_PATH))
        if os.environ.get("B200_GEMM_2CTA", "1") == "0":     # A/B switch: prefill GEMMs on the one-CTA kernel only
            _lib.b200_gemm_2cta_enable(0)
    return _lib


def stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    """Per-device int32 error word the kernels write on a bounded-wait expiry."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
        _status[idx] = t
    return t


def check_status(device=None) -> None:
    """Synchronising read of the error word; raises if any kernel recorded a timeout."""
    t = status_word(device)
    code = int(t.item())
    if code != 0:
        t.zero_()
        raise KernelError(f"device kernel reported error {code}: {ERR_NAMES.get(code, 'unknown')}")


LAUNCHES = 0  # kernels launched through this module (eager count; graph replays are added by the caller)


def check(rc: int, what: str, n_kernels: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += n_kernels
    if rc != 0:
        if rc < 0:
            raise KernelError(f"{what}: {ERR_NAMES.get(-rc, 'error')} ({rc})")
        raise KernelError(f"{what}: CUDA error {rc}")
