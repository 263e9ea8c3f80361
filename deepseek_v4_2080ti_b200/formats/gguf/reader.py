"""GGUF reader (v2/v3): header, metadata, tensor infos, mmap'ed raw tensor bytes, multi-shard bundles
(``name-00001-of-0000N.gguf``).  Behaviour follows src/loader/gguf/reader.py:121-204 and bundle.py:115-204."""
from __future__ import annotations

import mmap
import os
import re
import struct
from dataclasses import dataclass
from typing import Any

import torch

from .constants import BLOCK_BYTES, BLOCK_ELEMS, DEFAULT_ALIGNMENT, GGUF_MAGIC, GGMLType, ValueType
from .quant import dequantize

_SCALAR = {ValueType.UINT8: "<B", ValueType.INT8: "<b", ValueType.UINT16: "<H", ValueType.INT16: "<h",
           ValueType.UINT32: "<I", ValueType.INT32: "<i", ValueType.FLOAT32: "<f", ValueType.BOOL: "<?",
           ValueType.UINT64: "<Q", ValueType.INT64: "<q", ValueType.FLOAT64: "<d"}


@dataclass
class TensorInfo:
    name: str
    shape: tuple[int, ...]        # torch order: [..., rows, cols]
    ggml_type: GGMLType
    offset: int                   # from the start of the data section
    nbytes: int
    file: "GGUFFile | None" = None

    @property
    def cols(self) -> int:
        return self.shape[-1]

    @property
    def row_bytes(self) -> int:
        return self.cols // BLOCK_ELEMS[self.ggml_type] * BLOCK_BYTES[self.ggml_type]


class GGUFFile:
    def __init__(self, path: str):
        """A file that does not parse raises ``ValueError`` (whatever went wrong underneath: a short read, a count that
        does not fit, an unknown type code)."""
        self.path = path
        self._f = open(path, "rb")
        try:
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
            self._parse(path)
        except (struct.error, OverflowError, KeyError, IndexError, MemoryError) as exc:
            raise ValueError(f"{path}: malformed GGUF file ({type(exc).__name__}: {exc})") from exc

    def _parse(self, path: str) -> None:
        self._pos = 0
        magic, version = struct.unpack_from("<II", self._mm, 0)
        if magic != GGUF_MAGIC:
            raise ValueError(f"{path}: not a GGUF file")
        if version not in (2, 3):
            raise ValueError(f"{path}: unsupported GGUF version {version}")
        self.version = version
        n_tensors, n_kv = struct.unpack_from("<QQ", self._mm, 8)
        self._pos = 24
        self.metadata: dict[str, Any] = {}
        for _ in range(n_kv):
            k = self._string()
            vt = ValueType(self._unpack("<I"))
            self.metadata[k] = self._read_value(vt)
        self.alignment = int(self.metadata.get("general.alignment", DEFAULT_ALIGNMENT))
        self.tensors: dict[str, TensorInfo] = {}
        for _ in range(n_tensors):
            name = self._string()
            nd = self._unpack("<I")
            dims = [self._unpack("<Q") for _ in range(nd)]
            t = GGMLType(self._unpack("<I"))
            off = self._unpack("<Q")
            shape = tuple(reversed(dims))
            n_el = 1
            for d in shape:
                n_el *= d
            self.tensors[name] = TensorInfo(name, shape, t, off, n_el // BLOCK_ELEMS[t] * BLOCK_BYTES[t], self)
        self.data_start = (self._pos + self.alignment - 1) // self.alignment * self.alignment
        for ti in self.tensors.values():
            if self.data_start + ti.offset + ti.nbytes > len(self._mm):
                raise ValueError(f"{path}: tensor {ti.name} runs past the end of the file")

    def _unpack(self, fmt: str):
        (v,) = struct.unpack_from(fmt, self._mm, self._pos)
        self._pos += struct.calcsize(fmt)
        return v

    def _string(self) -> str:
        n = self._unpack("<Q")
        s = self._mm[self._pos:self._pos + n].decode("utf-8", errors="replace")
        self._pos += n
        return s

    def _read_value(self, vt: ValueType):
        if vt == ValueType.STRING:
            return self._string()
        if vt == ValueType.ARRAY:
            et = ValueType(self._unpack("<I"))
            n = self._unpack("<Q")
            return [self._read_value(et) for _ in range(n)]
        return self._unpack(_SCALAR[vt])

    def raw(self, name: str) -> torch.Tensor:
        """Raw block bytes of a tensor as ``uint8 [..., rows, row_bytes]`` (a view of the mapping, zero copy)."""
        ti = self.tensors[name]
        buf = torch.frombuffer(self._mm, dtype=torch.uint8, count=ti.nbytes, offset=self.data_start + ti.offset)
        return buf.view(*ti.shape[:-1], ti.row_bytes)

    def raw_expert(self, name: str, expert: int) -> torch.Tensor:
        """Slice ``expert`` of a stacked routed-expert tensor ``[experts, rows, cols]``."""
        ti = self.tensors[name]
        if len(ti.shape) != 3:
            raise ValueError(f"{name} is not a stacked expert tensor")
        return self.raw(name)[expert]

    def dequantized(self, name: str) -> torch.Tensor:
        ti = self.tensors[name]
        raw = self.raw(name).reshape(-1, ti.row_bytes)
        return dequantize(raw.clone(), ti.ggml_type, ti.cols).reshape(ti.shape)


_SHARD = re.compile(r"^(?P<stem>.*)-(?P<i>\d{5})-of-(?P<n>\d{5})\.gguf$")


class GGUFBundle:
    """One logical checkpoint over one or more shard files: merged metadata (first shard wins) and tensor index."""

    def __init__(self, files: list[GGUFFile]):
        self.files = files
        self.metadata: dict[str, Any] = {}
        self.tensors: dict[str, TensorInfo] = {}
        for f in reversed(files):
            self.metadata.update(f.metadata)
        for f in files:
            for k, ti in f.tensors.items():
                if k in self.tensors:
                    raise ValueError(f"tensor {k} appears in more than one shard")
                self.tensors[k] = ti

    @property
    def architecture(self) -> str:
        return str(self.metadata.get("general.architecture", ""))

    def raw(self, name: str) -> torch.Tensor:
        return self.tensors[name].file.raw(name)

    def dequantized(self, name: str) -> torch.Tensor:
        return self.tensors[name].file.dequantized(name)


def read_bundle(path: str) -> GGUFBundle:
    """``path``: a single ``.gguf`` file, any shard of a split checkpoint, or a directory holding the shards."""
    if os.path.isdir(path):
        names = sorted(n for n in os.listdir(path) if n.endswith(".gguf"))
        if not names:
            raise FileNotFoundError(f"no .gguf files in {path}")
        path = os.path.join(path, names[0])
    m = _SHARD.match(os.path.basename(path))
    if not m:
        return GGUFBundle([GGUFFile(path)])
    n = int(m.group("n"))
    d = os.path.dirname(path)
    files = []
    for i in range(1, n + 1):
        p = os.path.join(d, f"{m.group('stem')}-{i:05d}-of-{n:05d}.gguf")
        if not os.path.exists(p):
            raise FileNotFoundError(f"missing shard {p}")
        files.append(GGUFFile(p))
    return GGUFBundle(files)
