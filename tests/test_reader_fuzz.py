"""Malformed files: the Python readers answer with ValueError (never another exception type, never a hang), and the
native readers survive the same inputs - they run in a child process, so a crash shows as a signal instead of taking
the test session down."""
import os
import random
import struct
import subprocess
import sys

import pytest
import torch

from deepseek_v4_2080ti_b200.formats import safetensors_io, tensor_file
from deepseek_v4_2080ti_b200.formats.gguf import reader as gguf_reader
from deepseek_v4_2080ti_b200.models import v4_block_ref, v4_gguf

N = 120


def mutate(b: bytes, rng: random.Random) -> bytes:
    b = bytearray(b)
    kind = rng.choice(["trunc", "flip", "big", "zero"])
    if kind == "trunc":
        return bytes(b[:rng.randrange(0, len(b))])
    if kind == "flip":
        for _ in range(rng.randrange(1, 6)):
            b[rng.randrange(min(len(b), 3000))] ^= 1 << rng.randrange(8)
    else:
        i = rng.randrange(0, max(1, min(len(b) - 8, 400)))
        b[i:i + 8] = struct.pack("<Q", rng.choice([2 ** 63, 2 ** 64 - 1, 2 ** 40, 2 ** 32 + 5])) if kind == "big" else b"\0" * 8
    return bytes(b)


@pytest.fixture(scope="module")
def seeds(tmp_path_factory):
    d = tmp_path_factory.mktemp("seeds")
    cfg = v4_block_ref.V4Config(n_layers=1, compress_ratios=(4,), n_hash_layers=0, mtp=False, vocab_size=16, dim=32,
                                n_experts=2, moe_inter=16)
    v4_gguf.write_gguf(str(d / "s.gguf"), cfg, v4_block_ref.synth_weights(cfg, 0), "F32")
    safetensors_io.write_file(str(d / "s.safetensors"), {"a": torch.randn(4, 4), "b.c": torch.arange(6), "h": torch.randn(3).half()})
    tensor_file.write(d / "s.qdf2", tensor_file.TensorFile(1, 2, {"a": torch.randn(3, 3), "i": torch.arange(4)}))
    return {k: (d / f"s.{k}").read_bytes() for k in ("gguf", "safetensors", "qdf2")}


def _read_safetensors(path):
    f = safetensors_io.SafetensorsFile(path)
    for k in f.keys():
        f.get(k)


@pytest.mark.parametrize("kind,reader", [("gguf", gguf_reader.GGUFFile), ("safetensors", _read_safetensors), ("qdf2", tensor_file.read)])
def test_python_readers_raise_value_error_on_malformed_input(kind, reader, seeds, tmp_path):
    rng = random.Random(7)
    reader_ok = 0
    for i in range(N):
        p = str(tmp_path / f"case{i}")
        with open(p, "wb") as f:
            f.write(mutate(seeds[kind], rng))
        try:
            reader(p)
            reader_ok += 1
        except ValueError:
            pass                                                   # JSON and UTF-8 errors are ValueErrors too
    assert 0 < reader_ok < N                                       # the mutations hit both harmless and fatal bytes
    p = str(tmp_path / "intact")
    with open(p, "wb") as f:
        f.write(seeds[kind])
    reader(p)


CHILD = r"""
import os, sys
from deepseek_v4_2080ti_b200 import pocketllm_cpp as cpp
kind, d = sys.argv[1], sys.argv[2]
ok = err = 0
for f in sorted(os.listdir(d)):
    p = os.path.join(d, f)
    try:
        if kind == "gguf":
            r = cpp.GGUFReader(p)
            r.metadata()
            for t in list(r.tensor_names())[:4]:
                r.tensor_info(t); r.tensor_bytes(t)
        elif kind == "safetensors":
            w = cpp.WeightSource.open(p)
            for n in list(w.names())[:4]:
                w.get(n)
        else:
            cpp.json_roundtrip(open(p, "rb").read().decode("utf-8", "replace"))
        ok += 1
    except Exception:
        err += 1
print("done", ok, err)
"""


@pytest.mark.parametrize("kind", ["gguf", "safetensors", "json"])
def test_native_readers_survive_malformed_input(kind, seeds, tmp_path):
    rng = random.Random(11)
    seed = seeds[kind] if kind != "json" else b'{"a": [1, 2.5, "x\\u00e9", {"b": null, "c": true}], "d": {"e": -1e10}}'
    for i in range(N):
        data = seed if i == 0 else mutate(seed, rng)
        if kind == "safetensors":
            os.makedirs(tmp_path / f"c{i:03d}")
            (tmp_path / f"c{i:03d}" / "model.safetensors").write_bytes(data)
        else:
            (tmp_path / f"c{i:03d}").write_bytes(data)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", CHILD, kind, str(tmp_path)], capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, PYTHONPATH=root))
    assert r.returncode == 0, (r.returncode, r.stderr[-500:])         # a negative code is the signal that killed it
    _, ok, err = r.stdout.split()[-3:]
    assert int(ok) >= 1 and int(ok) + int(err) == N
