"""Flat named-tensor container used to exchange drafter fixtures (stage-by-stage activations of one proposal) between
an exporter and a checker.

Layout, little-endian: file header ``u32 magic "QDF2", u32 version = 1, i32 position_offset, i32 anchor_token,
u32 count``; then per record ``u32 name_len, u32 dtype (1 = f16, 2 = f32, 3 = i32), u32 ndim, u32 0, u64 nbytes``, the
UTF-8 name, ``ndim`` u64 extents and the C-order payload.  Scalars are not stored (``ndim >= 1``).

Same container as the reference's parity scripts read and write (cpp_engine/tests/qwen_dflash2_tensor_file.py:1-110),
so a fixture exported there from the upstream PyTorch drafter can be checked here.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np
import torch

MAGIC = int.from_bytes(b"QDF2", "little")
VERSION = 1
_FILE = struct.Struct("<IIiiI")
_REC = struct.Struct("<IIIIQ")
_CODES = {1: (np.dtype("<f2"), torch.float16), 2: (np.dtype("<f4"), torch.float32), 3: (np.dtype("<i4"), torch.int32)}


@dataclass
class TensorFile:
    position_offset: int = 0
    anchor_token: int = 0
    tensors: dict[str, torch.Tensor] = field(default_factory=dict)


def _code(t: torch.Tensor) -> int:
    if t.dtype in (torch.float16, torch.bfloat16):
        return 1
    if t.dtype in (torch.float32, torch.float64):
        return 2
    if t.dtype in (torch.int32, torch.int64, torch.uint8, torch.int16, torch.bool):
        return 3
    raise ValueError(f"tensor file cannot hold {t.dtype}")


def write(path: str | Path, f: TensorFile) -> int:
    """Returns the number of bytes written.  bf16 is stored as f16, f64 as f32, integers as i32."""
    with open(path, "wb") as out:
        out.write(_FILE.pack(MAGIC, VERSION, int(f.position_offset), int(f.anchor_token), len(f.tensors)))
        for name, t in f.tensors.items():
            raw = name.encode()
            if not raw or len(raw) > 4096 or t.dim() == 0 or t.dim() > 8:
                raise ValueError(f"invalid tensor record {name!r}")
            code = _code(t)
            arr = np.ascontiguousarray(t.detach().cpu().to(_CODES[code][1]).numpy().astype(_CODES[code][0], copy=False))
            out.write(_REC.pack(len(raw), code, arr.ndim, 0, arr.nbytes))
            out.write(raw)
            out.write(struct.pack(f"<{arr.ndim}Q", *arr.shape))
            out.write(arr.tobytes(order="C"))
        return out.tell()


def read(path: str | Path) -> TensorFile:
    data = Path(path).read_bytes()
    if len(data) < _FILE.size:
        raise ValueError(f"truncated tensor file header: {path}")
    magic, version, pos, anchor, count = _FILE.unpack_from(data, 0)
    if magic != MAGIC or version != VERSION:
        raise ValueError(f"not a version-{VERSION} tensor file: {path}")
    off, out = _FILE.size, TensorFile(pos, anchor)
    for _ in range(count):
        if off + _REC.size > len(data):
            raise ValueError(f"truncated tensor record header: {path}")
        name_len, code, ndim, reserved, nbytes = _REC.unpack_from(data, off)
        off += _REC.size
        if code not in _CODES or not 1 <= ndim <= 8 or reserved != 0 or not 1 <= name_len <= 4096:
            raise ValueError(f"malformed tensor record in {path}")
        name = data[off:off + name_len].decode()                          # a bad name is a UnicodeDecodeError, a ValueError
        off += name_len
        if off + 8 * ndim > len(data):
            raise ValueError(f"truncated tensor shape in {path}")
        shape = struct.unpack_from(f"<{ndim}Q", data, off)
        off += 8 * ndim
        np_dtype = _CODES[code][0]
        count = 1
        for d in shape:
            count *= int(d)                                              # Python integers: no wrap-around on hostile extents
        want = count * np_dtype.itemsize
        if want != nbytes or off + nbytes > len(data):
            raise ValueError(f"tensor {name!r}: payload size does not match its shape in {path}")
        if name in out.tensors:
            raise ValueError(f"tensor {name!r} appears twice in {path}")
        out.tensors[name] = torch.from_numpy(np.frombuffer(data, np_dtype, count, off).reshape(shape).copy())
        off += nbytes
    if off != len(data):
        raise ValueError(f"trailing bytes after the last record in {path}")
    return out
