"""ND4J data-type enum with the numeric ids used by the native array format.

The numeric values match ``libnd4j/include/array/DataType.h:27-52`` because they are
stored inside FlatBuffers graphs (``FlatArray.dtype``) and must survive a round trip.
The option bits used inside a shape-info buffer follow
``nd4j-api/.../linalg/api/shape/options/ArrayOptionsHelper.java:49-64``.
"""
from __future__ import annotations

import enum

import numpy as np
import torch


class DataType(enum.IntEnum):
    INHERIT = 0
    BOOL = 1
    FLOAT8 = 2
    HALF = 3
    HALF2 = 4
    FLOAT = 5
    DOUBLE = 6
    BYTE = 7      # INT8
    SHORT = 8     # INT16
    INT = 9       # INT32
    LONG = 10     # INT64
    UBYTE = 11
    UINT16 = 12
    UINT32 = 13
    UINT64 = 14
    QINT8 = 15
    QINT16 = 16
    BFLOAT16 = 17
    UTF8 = 50
    COMPRESSED = 99
    UNKNOWN = 100

    # ---- helpers -------------------------------------------------------
    def is_fp(self) -> bool:
        return self in (DataType.HALF, DataType.FLOAT, DataType.DOUBLE, DataType.BFLOAT16)

    def is_int(self) -> bool:
        return self in (DataType.BYTE, DataType.SHORT, DataType.INT, DataType.LONG,
                        DataType.UBYTE, DataType.UINT16, DataType.UINT32, DataType.UINT64)

    def width(self) -> int:
        return _WIDTH[self]

    def to_torch(self) -> torch.dtype:
        return _TO_TORCH[self]

    def to_numpy(self):
        return _TO_NUMPY[self]

    @staticmethod
    def from_torch(dt: torch.dtype) -> "DataType":
        return _FROM_TORCH[dt]

    @staticmethod
    def from_numpy(dt) -> "DataType":
        return _FROM_NUMPY[np.dtype(dt)]

    @staticmethod
    def from_name(name: str) -> "DataType":
        n = name.upper()
        alias = {"FLOAT32": "FLOAT", "FLOAT16": "HALF", "FLOAT64": "DOUBLE", "INT8": "BYTE", "INT16": "SHORT",
                 "INT32": "INT", "INT64": "LONG", "UINT8": "UBYTE", "BF16": "BFLOAT16"}
        return DataType[alias.get(n, n)]


_WIDTH = {DataType.BOOL: 1, DataType.FLOAT8: 1, DataType.HALF: 2, DataType.HALF2: 4, DataType.FLOAT: 4,
          DataType.DOUBLE: 8, DataType.BYTE: 1, DataType.SHORT: 2, DataType.INT: 4, DataType.LONG: 8,
          DataType.UBYTE: 1, DataType.UINT16: 2, DataType.UINT32: 4, DataType.UINT64: 8,
          DataType.QINT8: 1, DataType.QINT16: 2, DataType.BFLOAT16: 2, DataType.UTF8: 1,
          DataType.COMPRESSED: 1, DataType.UNKNOWN: 0, DataType.INHERIT: 0}

_TO_TORCH = {DataType.BOOL: torch.bool, DataType.HALF: torch.float16, DataType.FLOAT: torch.float32,
             DataType.DOUBLE: torch.float64, DataType.BYTE: torch.int8, DataType.SHORT: torch.int16,
             DataType.INT: torch.int32, DataType.LONG: torch.int64, DataType.UBYTE: torch.uint8,
             DataType.UINT16: torch.uint16, DataType.UINT32: torch.uint32, DataType.UINT64: torch.uint64,
             DataType.BFLOAT16: torch.bfloat16, DataType.FLOAT8: torch.float8_e4m3fn}
_FROM_TORCH = {v: k for k, v in _TO_TORCH.items()}

_TO_NUMPY = {DataType.BOOL: np.dtype(np.bool_), DataType.HALF: np.dtype(np.float16),
             DataType.FLOAT: np.dtype(np.float32), DataType.DOUBLE: np.dtype(np.float64),
             DataType.BYTE: np.dtype(np.int8), DataType.SHORT: np.dtype(np.int16),
             DataType.INT: np.dtype(np.int32), DataType.LONG: np.dtype(np.int64),
             DataType.UBYTE: np.dtype(np.uint8), DataType.UINT16: np.dtype(np.uint16),
             DataType.UINT32: np.dtype(np.uint32), DataType.UINT64: np.dtype(np.uint64),
             DataType.BFLOAT16: np.dtype(np.uint16)}  # numpy has no bf16: raw bits
_FROM_NUMPY = {v: k for k, v in _TO_NUMPY.items() if k != DataType.BFLOAT16}

# shape-info "extras" option bits
ATYPE_SPARSE_BIT = 2
ATYPE_COMPRESSED_BIT = 4
ATYPE_EMPTY_BIT = 8
DTYPE_BFLOAT16_BIT = 2048
DTYPE_HALF_BIT = 4096
DTYPE_FLOAT_BIT = 8192
DTYPE_DOUBLE_BIT = 16384
DTYPE_BYTE_BIT = 32768
DTYPE_SHORT_BIT = 65536
DTYPE_INT_BIT = 131072
DTYPE_LONG_BIT = 262144
DTYPE_BOOL_BIT = 524288
DTYPE_UTF8_BIT = 1048576
DTYPE_UNSIGNED_BIT = 8388608

_BITS = {DataType.HALF: DTYPE_HALF_BIT, DataType.BFLOAT16: DTYPE_BFLOAT16_BIT, DataType.FLOAT: DTYPE_FLOAT_BIT,
         DataType.DOUBLE: DTYPE_DOUBLE_BIT, DataType.INT: DTYPE_INT_BIT, DataType.LONG: DTYPE_LONG_BIT,
         DataType.BOOL: DTYPE_BOOL_BIT, DataType.BYTE: DTYPE_BYTE_BIT, DataType.SHORT: DTYPE_SHORT_BIT,
         DataType.UTF8: DTYPE_UTF8_BIT,
         DataType.UINT32: DTYPE_INT_BIT | DTYPE_UNSIGNED_BIT, DataType.UINT64: DTYPE_LONG_BIT | DTYPE_UNSIGNED_BIT,
         DataType.UBYTE: DTYPE_BYTE_BIT | DTYPE_UNSIGNED_BIT, DataType.UINT16: DTYPE_SHORT_BIT | DTYPE_UNSIGNED_BIT}


def extras_for(dtype: DataType, empty: bool = False) -> int:
    v = _BITS[dtype]
    if empty:
        v |= ATYPE_EMPTY_BIT
    return v


def dtype_from_extras(extras: int) -> DataType:
    unsigned = bool(extras & DTYPE_UNSIGNED_BIT)
    for dt, bits in _BITS.items():
        base = bits & ~DTYPE_UNSIGNED_BIT
        if extras & base and bool(bits & DTYPE_UNSIGNED_BIT) == unsigned:
            return dt
    raise ValueError(f"no data type bit in extras {extras}")
