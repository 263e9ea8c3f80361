"""Safetensors container I/O without the ``safetensors`` package: 8-byte little-endian header
length, JSON header (dtype / shape / data_offsets), raw payload.  Writes FP8 E4M3 / E8M0 / BF16 /
F32 / U8 tensors; reads through mmap; shards large checkpoints and writes
``model.safetensors.index.json`` like Hugging Face checkpoints
(reference: src/loader/safetensors.py:14-76, cpp_engine/core/safetensors_reader.cpp).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Iterable, Iterator

import torch

_DT = {torch.float8_e4m3fn: "F8_E4M3", torch.float8_e5m2: "F8_E5M2", torch.bfloat16: "BF16", torch.float16: "F16",
       torch.float32: "F32", torch.uint8: "U8", torch.int8: "I8", torch.int32: "I32", torch.int64: "I64"}
if hasattr(torch, "float8_e8m0fnu"):
    _DT[torch.float8_e8m0fnu] = "F8_E8M0"
_RD = {v: k for k, v in _DT.items()}


def _raw(t: torch.Tensor) -> bytes:
    t = t.detach().contiguous().cpu()
    return t.view(torch.uint8).numpy().tobytes() if t.numel() else b""


def write_file(path: str, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None) -> int:
    header: dict = {}
    if metadata:
        header["__metadata__"] = metadata
    off = 0
    blobs = []
    for name, t in tensors.items():
        if t.dtype not in _DT:
            raise ValueError(f"unsupported dtype {t.dtype} for {name}")
        b = _raw(t)
        header[name] = {"dtype": _DT[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
        off += len(b)
        blobs.append(b)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * ((-len(h)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)
    return off


def write_checkpoint(directory: str, state: Iterable[tuple[str, torch.Tensor]], shard_bytes: int = 4 << 30,
                     config_json: str | None = None) -> list[str]:
    """Stream (name, tensor) pairs into ``model-0000i.safetensors`` shards + index (+ config.json).
    A shard is written as soon as it is full, so host memory holds one shard at a time."""
    os.makedirs(directory, exist_ok=True)
    files: list[str] = []
    weight_map: dict[str, str] = {}
    total = 0
    cur: dict[str, torch.Tensor] = {}
    size = 0

    def flush() -> None:
        nonlocal cur, size, total
        if not cur:
            return
        fn = f"model-{len(files) + 1:05d}.safetensors"
        total += write_file(os.path.join(directory, fn), cur, {"format": "pt"})
        files.append(fn)
        for k in cur:
            weight_map[k] = fn
        cur, size = {}, 0

    for name, t in state:
        n = t.numel() * t.element_size()
        if size and size + n > shard_bytes:
            flush()
        cur[name] = t.cpu()
        size += n
    flush()
    if len(files) == 1:
        os.replace(os.path.join(directory, files[0]), os.path.join(directory, "model.safetensors"))
        files = ["model.safetensors"]
        weight_map = {k: "model.safetensors" for k in weight_map}
    with open(os.path.join(directory, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f)
    if config_json is not None:
        with open(os.path.join(directory, "config.json"), "w") as f:
            f.write(config_json)
    return files


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        if len(self._mm) < 8:
            raise ValueError(f"{path}: too short for a safetensors file")
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if hlen <= 0 or hlen > len(self._mm) - 8:
            raise ValueError(f"bad safetensors header length in {path}")
        self.header = json.loads(self._mm[8:8 + hlen].decode())          # JSON / UTF-8 errors are ValueErrors
        if not isinstance(self.header, dict):
            raise ValueError(f"{path}: the safetensors header is not an object")
        self.metadata = self.header.pop("__metadata__", {})
        self._base = 8 + hlen
        size = len(self._mm) - self._base
        for name, info in self.header.items():                           # every record checked once, here
            try:
                b, e = (int(v) for v in info["data_offsets"])
                n = 1
                for d in info["shape"]:
                    n *= int(d)
                dt = _RD.get(info["dtype"])                           # a dtype this reader has no tensor type for is
                item = torch.empty((), dtype=dt).element_size() if dt is not None else None   # refused when it is read
            except (KeyError, TypeError, ValueError) as exc:
                raise ValueError(f"{path}: malformed record for tensor {name!r}") from exc
            if not 0 <= b <= e <= size or (item is not None and (e - b) != n * item):
                raise ValueError(f"{path}: tensor {name!r} does not fit its bytes ({b}..{e} of {size}, shape {info['shape']})")

    def keys(self) -> list[str]:
        return list(self.header)

    def get(self, name: str) -> torch.Tensor:
        info = self.header[name]
        b, e = info["data_offsets"]
        if info["dtype"] not in _RD:
            raise ValueError(f"{self.path}: tensor {name!r} has dtype {info['dtype']}, which this reader does not map")
        dt = _RD[info["dtype"]]
        buf = torch.frombuffer(self._mm, dtype=torch.uint8, count=e - b, offset=self._base + b) if e > b else torch.empty(0, dtype=torch.uint8)
        return buf.view(dt).reshape(info["shape"])


def read_checkpoint(directory: str) -> Iterator[tuple[str, torch.Tensor]]:
    """Yield (name, tensor) from every shard of a checkpoint directory (index order when an index exists)."""
    idx = os.path.join(directory, "model.safetensors.index.json")
    if os.path.exists(idx):
        wm = json.load(open(idx))["weight_map"]
        files: dict[str, SafetensorsFile] = {}
        for name, fn in wm.items():
            if fn not in files:
                files[fn] = SafetensorsFile(os.path.join(directory, fn))
            yield name, files[fn].get(name)
    else:
        for fn in sorted(os.listdir(directory)):
            if fn.endswith(".safetensors"):
                f = SafetensorsFile(os.path.join(directory, fn))
                for name in f.keys():
                    yield name, f.get(name)
