"""Guard bands around workspaces: with no memory checker available on the GPU, a kernel that writes a little past (or
before) the buffer it was given is caught by the bytes next to it.

``empty(...)`` is ``torch.empty`` when guards are off (the default).  With ``B200_CANARY=1`` in the environment, or
inside ``enabled(True)``, it allocates ``band + payload + band`` bytes, fills both bands with a fixed pattern and
returns the payload as a tensor of the requested shape; the allocation is remembered (weakly: it leaves the registry
when the tensor dies) and ``verify_all()`` reports every band whose pattern was disturbed, with the buffer's name, the
side and the first bad offset.  The tests verify after every GPU test (tests/conftest.py); the symmetric buffers of
the peer-memory communicator carry the same bands (``parallel/tp.py``).

The reference has no counterpart (it relies on overwrite-safety tests, cpp_engine/tests/test_verify_overwrite_safety.cpp);
this is the stand-in for a device memory checker on hosts where none can be run.
"""
from __future__ import annotations

import contextlib
import os
import weakref
from dataclasses import dataclass

import torch

PATTERN = 0xA5
DEFAULT_BAND = 4096          # bytes on each side; a multiple of 256 keeps the payload's alignment

_forced: bool | None = None
_registry: "dict[int, _Guarded]" = {}
_next_id = 0


def is_enabled() -> bool:
    return _forced if _forced is not None else os.environ.get("B200_CANARY", "0") == "1"


@contextlib.contextmanager
def enabled(on: bool = True):
    global _forced
    prev, _forced = _forced, on
    try:
        yield
    finally:
        _forced = prev


@dataclass
class Violation:
    name: str
    side: str                 # "before" | "after"
    offset: int               # first disturbed byte, counted from the start of that band
    count: int                # disturbed bytes in the band
    value: int                # what the first disturbed byte holds now

    def __str__(self) -> str:
        return f"{self.name}: {self.count} byte(s) {self.side} the buffer overwritten, first at +{self.offset} (now 0x{self.value:02x})"


class _Guarded:
    def __init__(self, name: str, raw: torch.Tensor, band: int, nbytes: int):
        self.name, self.raw, self.band, self.nbytes = name, raw, band, nbytes


def empty(*shape, dtype=torch.float32, device=None, name: str = "", band: int = DEFAULT_BAND) -> torch.Tensor:
    """``torch.empty`` with guard bands when guards are on.  ``shape`` as ints or one tuple."""
    global _next_id
    if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
        shape = tuple(shape[0])
    if not is_enabled():
        return torch.empty(*shape, dtype=dtype, device=device)
    numel = 1
    for d in shape:
        numel *= int(d)
    item = torch.empty((), dtype=dtype).element_size()
    nbytes = numel * item
    pad = (-nbytes) % 256                   # keep the trailing band aligned; the pad belongs to the band
    raw = torch.empty(band + nbytes + pad + band, dtype=torch.uint8, device=device)
    g = _Guarded(name or f"buffer#{_next_id}", raw, band, nbytes)
    raw[:band].fill_(PATTERN)
    raw[band + nbytes:].fill_(PATTERN)          # the alignment pad is part of the trailing band
    view = raw[band:band + nbytes].view(dtype).view(*shape)
    key = _next_id
    _next_id += 1
    _registry[key] = g
    weakref.finalize(view, _registry.pop, key, None)
    return view


def zeros(*shape, dtype=torch.float32, device=None, name: str = "", band: int = DEFAULT_BAND) -> torch.Tensor:
    if not is_enabled():
        if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
            shape = tuple(shape[0])
        return torch.zeros(*shape, dtype=dtype, device=device)
    return empty(*shape, dtype=dtype, device=device, name=name, band=band).zero_()


def _check(g: _Guarded) -> list[Violation]:
    out = []
    before = g.raw[:g.band]
    after = g.raw[g.band + g.nbytes:]
    for side, b in (("before", before), ("after", after)):
        bad = (b != PATTERN).nonzero()
        if bad.numel():
            first = int(bad[0])
            out.append(Violation(g.name, side, first, int(bad.numel()), int(b[first])))
    return out


def verify_all(repaint: bool = True) -> list[Violation]:
    """Check every live guarded buffer; disturbed bands are repainted so that one overrun is reported once."""
    out: list[Violation] = []
    for g in list(_registry.values()):
        v = _check(g)
        if v and repaint:
            g.raw[:g.band].fill_(PATTERN)
            g.raw[g.band + g.nbytes:].fill_(PATTERN)
        out += v
    return out


def live_buffers() -> int:
    return len(_registry)


def assert_clean() -> None:
    v = verify_all()
    if v:
        raise AssertionError("guard bands disturbed:\n  " + "\n  ".join(str(x) for x in v))
