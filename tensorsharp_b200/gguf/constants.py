"""GGUF file-format constants: magic, value types, tensor types, block geometry.

Parity: TensorSharp.Runtime/GgufReader.cs:20-37 (type enums), :303-369 (block and
type sizes). The numeric values are fixed by the GGUF specification.
"""
from __future__ import annotations

import enum

GGUF_MAGIC = 0x46554747  # "GGUF" little endian
GGUF_VERSION = 3
GGUF_DEFAULT_ALIGNMENT = 32


class GGUFValueType(enum.IntEnum):
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


class GGMLType(enum.IntEnum):
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q4_1 = 3
    Q5_0 = 6
    Q5_1 = 7
    Q8_0 = 8
    Q8_1 = 9
    Q2_K = 10
    Q3_K = 11
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14
    Q8_K = 15
    IQ2_XXS = 16
    IQ2_XS = 17
    IQ3_XXS = 18
    IQ1_S = 19
    IQ4_NL = 20
    IQ3_S = 21
    IQ2_S = 22
    IQ4_XS = 23
    I8 = 24
    I16 = 25
    I32 = 26
    I64 = 27
    F64 = 28
    IQ1_M = 29
    BF16 = 30
    TQ1_0 = 34
    TQ2_0 = 35
    MXFP4 = 39


# (values per block, bytes per block)
_GEOMETRY = {
    GGMLType.F32: (1, 4),
    GGMLType.F16: (1, 2),
    GGMLType.BF16: (1, 2),
    GGMLType.F64: (1, 8),
    GGMLType.I8: (1, 1),
    GGMLType.I16: (1, 2),
    GGMLType.I32: (1, 4),
    GGMLType.I64: (1, 8),
    GGMLType.Q4_0: (32, 18),
    GGMLType.Q4_1: (32, 20),
    GGMLType.Q5_0: (32, 22),
    GGMLType.Q5_1: (32, 24),
    GGMLType.Q8_0: (32, 34),
    GGMLType.Q8_1: (32, 36),
    GGMLType.IQ4_NL: (32, 18),
    GGMLType.MXFP4: (32, 17),
    GGMLType.Q2_K: (256, 84),
    GGMLType.Q3_K: (256, 110),
    GGMLType.Q4_K: (256, 144),
    GGMLType.Q5_K: (256, 176),
    GGMLType.Q6_K: (256, 210),
    GGMLType.Q8_K: (256, 292),
    GGMLType.IQ2_XXS: (256, 66),
    GGMLType.IQ2_XS: (256, 74),
    GGMLType.IQ3_XXS: (256, 98),
    GGMLType.IQ1_S: (256, 50),
    GGMLType.IQ3_S: (256, 110),
    GGMLType.IQ2_S: (256, 82),
    GGMLType.IQ4_XS: (256, 136),
    GGMLType.IQ1_M: (256, 56),
    GGMLType.TQ1_0: (256, 54),
    GGMLType.TQ2_0: (256, 66),
}


def block_size(t: GGMLType) -> int:
    """Number of logical values stored in one block of type ``t``."""
    return _GEOMETRY[GGMLType(t)][0]


def type_size(t: GGMLType) -> int:
    """Bytes occupied by one block of type ``t``."""
    return _GEOMETRY[GGMLType(t)][1]


def row_bytes(t: GGMLType, ne0: int) -> int:
    """Bytes of one row of ``ne0`` values (``ne0`` must be a whole number of blocks)."""
    bs, ts = _GEOMETRY[GGMLType(t)]
    if ne0 % bs:
        raise ValueError(f"row length {ne0} is not a multiple of the {t.name} block size {bs}")
    return (ne0 // bs) * ts


def tensor_bytes(t: GGMLType, shape_ne) -> int:
    """Total bytes of a tensor whose GGUF dims (ne0 first) are ``shape_ne``."""
    n = 1
    for d in shape_ne[1:]:
        n *= int(d)
    return row_bytes(t, int(shape_ne[0])) * n


# Types whose blocks the device kernels consume directly (no load-time dequantisation).
DEVICE_QUANT_TYPES = (
    GGMLType.Q4_0, GGMLType.Q8_0, GGMLType.Q4_K, GGMLType.Q5_K, GGMLType.Q6_K, GGMLType.MXFP4,
)
