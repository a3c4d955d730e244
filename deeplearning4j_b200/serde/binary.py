"""ND4J binary array stream (``Nd4j.write`` / ``Nd4j.read``), bit-exact.

Layout (all big-endian, Java ``DataOutputStream``), from
``nd4j-api/.../linalg/factory/Nd4j.java:2764-2774`` and
``nd4j-api/.../linalg/api/buffer/BaseDataBuffer.java:1983-2028``::

    shapeInfo buffer : writeUTF(allocationMode) writeLong(length) writeUTF("LONG") length x int64
    data buffer      : writeUTF(allocationMode) writeLong(length) writeUTF(dtype)  length x element

``shapeInfo = [rank, shape.., stride.., extras, ews, order-char]``.  HALF and BFLOAT16 elements
travel as 16-bit patterns.  Data is written in the array's own ordering ('c' or 'f'), views
are materialised first.
"""
from __future__ import annotations

import io
import struct
from typing import BinaryIO

import numpy as np
import torch

from ..nd.dtype import DataType, dtype_from_extras, extras_for
from ..nd.ndarray import INDArray, _c_strides, _f_strides

ALLOCATION_MODE = "MIXED_DATA_TYPES"
_LEGACY_MODES = ("DIRECT", "HEAP", "JAVACPP", "LONG_SHAPE", "MIXED_DATA_TYPES")


def _write_utf(out: BinaryIO, s: str):
    b = s.encode("utf-8")  # names are ASCII; Java modified-UTF8 == UTF-8 for them
    out.write(struct.pack(">H", len(b)))
    out.write(b)


def _read_utf(inp: BinaryIO) -> str:
    (n,) = struct.unpack(">H", inp.read(2))
    return inp.read(n).decode("utf-8")


_BE = {DataType.DOUBLE: ">f8", DataType.FLOAT: ">f4", DataType.HALF: ">u2", DataType.BFLOAT16: ">u2",
       DataType.LONG: ">i8", DataType.UINT64: ">u8", DataType.INT: ">i4", DataType.UINT32: ">u4",
       DataType.SHORT: ">i2", DataType.UINT16: ">u2", DataType.BYTE: "i1", DataType.UBYTE: "u1", DataType.BOOL: "u1"}


def _flat_numpy(arr: INDArray, order: str) -> np.ndarray:
    t = arr.t.detach()
    if order == "f" and t.dim() > 1:
        t = t.permute(*reversed(range(t.dim())))
    t = t.contiguous().reshape(-1).cpu()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.bool:
        return t.to(torch.uint8).numpy()
    return t.numpy()


def write_buffer(out: BinaryIO, values: np.ndarray, dtype: DataType):
    _write_utf(out, ALLOCATION_MODE)
    out.write(struct.pack(">q", int(values.size)))
    _write_utf(out, dtype.name)
    out.write(np.ascontiguousarray(values).astype(_BE[dtype], copy=False).tobytes())


def read_buffer(inp: BinaryIO):
    mode = _read_utf(inp)
    if mode not in _LEGACY_MODES:
        raise ValueError(f"bad allocation mode {mode!r}")
    (length,) = struct.unpack(">q", inp.read(8))
    dtype = DataType.from_name(_read_utf(inp))
    if dtype == DataType.COMPRESSED:
        raise NotImplementedError("compressed buffers are handled by serde.compression")
    be = np.dtype(_BE[dtype])
    raw = inp.read(length * be.itemsize)
    if len(raw) != length * be.itemsize:
        raise EOFError("truncated ND4J buffer")
    return np.frombuffer(raw, dtype=be, count=length), dtype


def write_array(arr: INDArray, out: BinaryIO):
    """``Nd4j.write(INDArray, DataOutputStream)``."""
    arr = arr if isinstance(arr, INDArray) else INDArray(arr)
    order = arr.ordering()
    dtype = arr.dataType()
    shape = list(arr.shape())
    stride = _f_strides(shape) if order == "f" else _c_strides(shape)
    empty = arr.length() == 0
    info = [len(shape)] + shape + stride + [extras_for(dtype, empty), 1, ord(order)]
    write_buffer(out, np.asarray(info, dtype=np.int64), DataType.LONG)
    if not empty:
        write_buffer(out, _flat_numpy(arr, order), dtype)


def read_array(inp: BinaryIO, device=None) -> INDArray:
    """``Nd4j.read(DataInputStream)``."""
    info, it = read_buffer(inp)
    info = [int(v) for v in info]
    rank = info[0]
    shape = info[1:1 + rank]
    extras = info[1 + 2 * rank]
    order = chr(info[-1]) if info[-1] in (99, 102) else "c"
    n = int(np.prod(shape)) if rank else 1
    if extras & 8 or n == 0:
        dtype = dtype_from_extras(extras)
        return INDArray(torch.zeros(shape, dtype=dtype.to_torch(), device=device))
    vals, dtype = read_buffer(inp)
    native = vals.astype(vals.dtype.newbyteorder("="))
    if dtype in (DataType.HALF, DataType.BFLOAT16):
        t = torch.from_numpy(native.view(np.int16).copy()).view(dtype.to_torch())
    elif dtype == DataType.BOOL:
        t = torch.from_numpy(native.copy()).to(torch.bool)
    else:
        t = torch.from_numpy(native.copy())
    if device is not None:
        t = t.to(device)
    if order == "f" and rank > 1:
        t = t.reshape(tuple(reversed(shape))).permute(*reversed(range(rank)))
        return INDArray(t, "f")
    return INDArray(t.reshape(shape), "c")


def to_bytes(arr: INDArray) -> bytes:
    bio = io.BytesIO()
    write_array(arr, bio)
    return bio.getvalue()


def from_bytes(b: bytes, device=None) -> INDArray:
    return read_array(io.BytesIO(b), device)
