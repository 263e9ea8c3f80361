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
    7: "index out of range",
}

# sites of the debug index checks (B200_BOUNDS_CHECK=1), as recorded in the second byte of the error word
BOUNDS_SITES = {1: "token ids", 2: "kv cache element offsets", 3: "page table", 4: "state slots", 5: "selected key rows",
                6: "expert ids", 7: "logit rows"}


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
        if code & 0xFF == 7:
            site, pos = (code >> 8) & 0xFF, (code >> 16) & 0xFFFF
            raise KernelError(f"index out of range in {BOUNDS_SITES.get(site, f'site {site}')} at element "
                              f"{pos}{'+' if pos == 0xFFFF else ''} (the index was replaced by a valid one before the kernel ran)")
        raise KernelError(f"device kernel reported error {code}: {ERR_NAMES.get(code, 'unknown')}")


def bounds_checks_on() -> bool:
    return os.environ.get("B200_BOUNDS_CHECK", "0") == "1"


def check_indices(idx: torch.Tensor | None, lo: int, hi: int, site: int, keep: int | None = None) -> None:
    """Debug mode only (``B200_BOUNDS_CHECK=1``): scan an int32 index tensor on the device before the kernel that
    addresses memory through it; values outside ``[lo, hi)`` (other than the sentinel ``keep``) set the error word and
    are replaced by ``lo``.  No-op otherwise."""
    if idx is None or not bounds_checks_on() or idx.numel() == 0:
        return
    assert idx.dtype == torch.int32 and idx.is_cuda and idx.is_contiguous()
    rc = lib().b200_check_indices(ptr(idx), ctypes.c_longlong(idx.numel()), int(lo), int(hi), int(keep or 0),
                                  int(keep is not None), int(lo), ptr(status_word(idx.device)), int(site), stream())
    check(rc, "check_indices")


LAUNCHES = 0  # kernels launched through this module (eager count; graph replays are added by the caller)


def check(rc: int, what: str, n_kernels: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += n_kernels
    if rc != 0:
        if rc < 0:
            raise KernelError(f"{what}: {ERR_NAMES.get(-rc, 'error')} ({rc})")
        raise KernelError(f"{what}: CUDA error {rc}")
