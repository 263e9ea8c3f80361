"""GGUF v3 writer: metadata key/values, tensor infos, aligned tensor data
(container layout as parsed by src/loader/gguf/reader.py:121-204 and cpp_engine/core/gguf_reader.cpp)."""
from __future__ import annotations

import struct
from typing import Any, Iterable, Mapping

import torch

from .constants import BLOCK_BYTES, BLOCK_ELEMS, DEFAULT_ALIGNMENT, GGUF_MAGIC, GGUF_VERSION, GGMLType, ValueType


def _str(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


_SCALAR = {ValueType.UINT8: "<B", ValueType.INT8: "<b", ValueType.UINT16: "<H", ValueType.INT16: "<h",
           ValueType.UINT32: "<I", ValueType.INT32: "<i", ValueType.FLOAT32: "<f", ValueType.BOOL: "<?",
           ValueType.UINT64: "<Q", ValueType.INT64: "<q", ValueType.FLOAT64: "<d"}


def _vtype(v: Any) -> ValueType:
    if isinstance(v, bool):
        return ValueType.BOOL
    if isinstance(v, int):
        return ValueType.UINT32 if 0 <= v < 2 ** 32 else ValueType.INT64
    if isinstance(v, float):
        return ValueType.FLOAT32
    if isinstance(v, str):
        return ValueType.STRING
    if isinstance(v, (list, tuple)):
        return ValueType.ARRAY
    raise TypeError(f"unsupported GGUF metadata value {type(v)}")


def _value(v: Any, vt: ValueType | None = None) -> bytes:
    vt = vt or _vtype(v)
    if vt == ValueType.STRING:
        return _str(v)
    if vt == ValueType.ARRAY:
        et = _vtype(v[0]) if len(v) else ValueType.UINT32
        if et == ValueType.UINT32 and any(isinstance(x, int) and x < 0 for x in v):
            et = ValueType.INT32
        return struct.pack("<IQ", int(et), len(v)) + b"".join(_value(x, et) for x in v)
    return struct.pack(_SCALAR[vt], v)


def write_gguf(path: str, metadata: Mapping[str, Any], tensors: Iterable[tuple[str, torch.Tensor, GGMLType, tuple[int, ...]]],
               alignment: int = DEFAULT_ALIGNMENT) -> None:
    """tensors: (name, raw uint8 data as produced by ``quantize`` (any shape), ggml type, logical shape with the
    row-major torch convention ``[..., rows, cols]``).  GGUF stores dims innermost first."""
    tensors = list(tensors)
    meta = dict(metadata)
    meta.setdefault("general.alignment", alignment)
    head = struct.pack("<IIQQ", GGUF_MAGIC, GGUF_VERSION, len(tensors), len(meta))
    kv = b""
    for k, v in meta.items():
        vt = _vtype(v)
        kv += _str(k) + struct.pack("<I", int(vt)) + _value(v, vt)
    infos = b""
    off = 0
    offsets = []
    for name, raw, t, shape in tensors:
        t = GGMLType(t)
        n_el = 1
        for d in shape:
            n_el *= d
        nbytes = n_el // BLOCK_ELEMS[t] * BLOCK_BYTES[t]
        if raw.numel() * raw.element_size() != nbytes:
            raise ValueError(f"{name}: {raw.numel() * raw.element_size()} bytes given, {nbytes} expected for {t.name} {shape}")
        dims = list(reversed(shape))
        infos += _str(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", int(t), off)
        offsets.append(off)
        off += (nbytes + alignment - 1) // alignment * alignment
    pre = head + kv + infos
    pad = (-len(pre)) % alignment
    with open(path, "wb") as f:
        f.write(pre + b"\0" * pad)
        base = f.tell()
        for (name, raw, t, shape), o in zip(tensors, offsets):
            f.seek(base + o)
            f.write(raw.detach().contiguous().cpu().view(torch.uint8).numpy().tobytes())
        f.truncate(base + off)       # zero padding after the last tensor up to the alignment
