"""ggml tensor type ids, block geometry, and metadata value types of the GGUF container
(same table as the reference's src/loader/gguf/reader.py:27-57; kernel type ids as
src/loader/gguf/quant_types.py:3-13)."""
from __future__ import annotations

import enum

GGUF_MAGIC = 0x46554747      # "GGUF" little endian
GGUF_VERSION = 3
DEFAULT_ALIGNMENT = 32
QK_K = 256


class GGMLType(enum.IntEnum):
    F32 = 0
    F16 = 1
    Q8_0 = 8
    Q2_K = 10
    Q3_K = 11
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14
    IQ2_XXS = 16
    IQ2_XS = 17
    IQ3_XXS = 18
    IQ4_XS = 23
    I8 = 24
    I32 = 26
    IQ1_M = 29
    BF16 = 30


BLOCK_ELEMS = {GGMLType.F32: 1, GGMLType.F16: 1, GGMLType.BF16: 1, GGMLType.I8: 1, GGMLType.I32: 1,
               GGMLType.Q8_0: 32, GGMLType.Q2_K: 256, GGMLType.Q3_K: 256, GGMLType.Q4_K: 256, GGMLType.Q5_K: 256,
               GGMLType.Q6_K: 256, GGMLType.IQ2_XXS: 256, GGMLType.IQ2_XS: 256, GGMLType.IQ3_XXS: 256,
               GGMLType.IQ4_XS: 256, GGMLType.IQ1_M: 256}
BLOCK_BYTES = {GGMLType.F32: 4, GGMLType.F16: 2, GGMLType.BF16: 2, GGMLType.I8: 1, GGMLType.I32: 4,
               GGMLType.Q8_0: 34, GGMLType.Q2_K: 84, GGMLType.Q3_K: 110, GGMLType.Q4_K: 144, GGMLType.Q5_K: 176,
               GGMLType.Q6_K: 210, GGMLType.IQ2_XXS: 66, GGMLType.IQ2_XS: 74, GGMLType.IQ3_XXS: 98,
               GGMLType.IQ4_XS: 136, GGMLType.IQ1_M: 56}

# ids the fused kernels switch on
KERNEL_TYPE_ID = {GGMLType.IQ2_XXS: 0, GGMLType.Q2_K: 1, GGMLType.IQ1_M: 2, GGMLType.Q4_K: 3, GGMLType.Q5_K: 4,
                  GGMLType.IQ2_XS: 5, GGMLType.IQ3_XXS: 6, GGMLType.IQ4_XS: 7, GGMLType.Q6_K: 8, GGMLType.Q8_0: 9}


class ValueType(enum.IntEnum):
    UINT8 = 0
    INT8 = 1
    UINT16 = 2
    INT16 = 3
    UINT32 = 4
    INT32 = 5
    FLOAT32 = 6
    BOOL = 7
    STRING = 8
    ARRAY = 9
    UINT64 = 10
    INT64 = 11
    FLOAT64 = 12


def row_bytes(t: GGMLType, n_cols: int) -> int:
    be = BLOCK_ELEMS[t]
    if n_cols % be:
        raise ValueError(f"{t.name}: row length {n_cols} is not a multiple of the block size {be}")
    return n_cols // be * BLOCK_BYTES[t]
