"""NDArray compression SPI (``nd4j-api/.../linalg/compression``): ``BasicNDArrayCompressor`` with the
GZIP, NOOP, INT8, FLOAT16 / FLOAT8-style codecs and the gradient codecs THRESHOLD / BITMAP
(``CpuThreshold`` / ``CudaThreshold``: ``nd4j-cuda/.../compression/CudaThreshold.java:48-139``).

A compressed array is a ``CompressedArray`` (descriptor + payload), the stand-in for an INDArray whose
buffer is a ``CompressedDataBuffer`` with a ``CompressionDescriptor``.
"""
from __future__ import annotations

import gzip
from dataclasses import dataclass

import numpy as np
import torch

from ..nd.dtype import DataType
from ..nd.ndarray import INDArray
from ..parallel import codec as gradcodec


class CompressionType:
    LOSSY = "LOSSY"
    LOSSLESS = "LOSSLESS"


@dataclass
class CompressionDescriptor:
    compressionAlgorithm: str
    compressionType: str
    originalLength: int          # bytes
    compressedLength: int        # bytes
    numberOfElements: int
    originalElementSize: int
    originalDataType: DataType
    shape: tuple = ()


class CompressedArray:
    def __init__(self, descriptor, payload, extra=None):
        self.descriptor, self.payload, self.extra = descriptor, payload, extra or {}

    def isCompressed(self): return True
    def shape(self): return list(self.descriptor.shape)
    def compressionRatio(self): return self.descriptor.originalLength / max(self.descriptor.compressedLength, 1)


def _t(x):
    return x.t if isinstance(x, INDArray) else x


class NDArrayCompressor:
    NAME = ""
    TYPE = CompressionType.LOSSLESS
    def getDescriptor(self): return self.NAME
    def getCompressionType(self): return self.TYPE
    def configure(self, *args): pass

    def _desc(self, t, nbytes):
        return CompressionDescriptor(self.NAME, self.TYPE, t.numel() * t.element_size(), nbytes, t.numel(), t.element_size(),
                                     DataType.from_torch(t.dtype), tuple(t.shape))


class NoOp(NDArrayCompressor):
    NAME = "NOOP"
    def compress(self, arr):
        t = _t(arr).detach().contiguous()
        return CompressedArray(self._desc(t, t.numel() * t.element_size()), t.clone())
    def decompress(self, c): return INDArray(c.payload.clone())


class Gzip(NDArrayCompressor):
    NAME = "GZIP"
    def compress(self, arr):
        t = _t(arr).detach().contiguous().cpu()
        raw = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        z = gzip.compress(raw, 6)
        return CompressedArray(self._desc(t, len(z)), z)

    def decompress(self, c):
        d = c.descriptor
        raw = gzip.decompress(c.payload)
        tdt = d.originalDataType.to_torch()
        if tdt == torch.bfloat16:
            t = torch.from_numpy(np.frombuffer(raw, dtype=np.int16).copy()).view(torch.bfloat16)
        else:
            t = torch.from_numpy(np.frombuffer(raw, dtype=torch.empty(0, dtype=tdt).numpy().dtype).copy())
        return INDArray(t.reshape(d.shape))


class Float16(NDArrayCompressor):
    NAME, TYPE = "FLOAT16", CompressionType.LOSSY
    def compress(self, arr):
        t = _t(arr).detach()
        h = t.to(torch.float16).contiguous()
        return CompressedArray(self._desc(t, h.numel() * 2), h)
    def decompress(self, c): return INDArray(c.payload.to(c.descriptor.originalDataType.to_torch()))


class Int8(NDArrayCompressor):
    """Linear 8-bit quantisation with a (min, max) header (``convertToQuantized`` in the native type-conversion code)."""
    NAME, TYPE = "INT8", CompressionType.LOSSY
    def compress(self, arr):
        t = _t(arr).detach().float()
        lo, hi = float(t.min()), float(t.max())
        scale = (hi - lo) / 255.0 if hi > lo else 1.0
        q = ((t - lo) / scale).round().clamp(0, 255).to(torch.uint8)
        return CompressedArray(self._desc(_t(arr), q.numel() + 8), q, {"min": lo, "max": hi})
    def decompress(self, c):
        lo, hi = c.extra["min"], c.extra["max"]
        scale = (hi - lo) / 255.0 if hi > lo else 1.0
        return INDArray((c.payload.float() * scale + lo).to(c.descriptor.originalDataType.to_torch()))


class Threshold(NDArrayCompressor):
    """Sparse threshold encoding of a gradient-like array.  ``compress`` subtracts the encoded part from the
    input in place (the residual stays behind), exactly as the gradient-sharing path uses it; returns ``None``
    when nothing reaches the threshold."""
    NAME, TYPE = "THRESHOLD", CompressionType.LOSSY

    def __init__(self, threshold=1e-3): self.threshold = float(threshold)
    def configure(self, *args):
        if args:
            self.threshold = float(args[0])

    def compress(self, arr, boundary=None):
        t = _t(arr)
        flat = t.reshape(-1)
        msg = gradcodec.threshold_encode(flat, self.threshold, boundary)
        if int(msg[0]) == 0:
            return None
        return CompressedArray(self._desc(t, msg.numel() * 4), msg)

    def decompress(self, c, target=None):
        d = c.descriptor
        out = _t(target) if target is not None else torch.zeros(d.shape, dtype=torch.float32, device=c.payload.device)
        gradcodec.threshold_decode(c.payload, out.reshape(-1))
        return INDArray(out) if target is None else target


class Bitmap(Threshold):
    NAME = "BITMAP"
    def compress(self, arr, boundary=None):
        t = _t(arr)
        msg = gradcodec.bitmap_encode(t.reshape(-1), self.threshold)
        return CompressedArray(self._desc(t, msg.numel() * 4), msg)

    def decompress(self, c, target=None):
        d = c.descriptor
        out = _t(target) if target is not None else torch.zeros(d.shape, dtype=torch.float32, device=c.payload.device)
        gradcodec.bitmap_decode(c.payload, out.reshape(-1))
        return INDArray(out) if target is None else target


class BasicNDArrayCompressor:
    """Registry + default algorithm (``BasicNDArrayCompressor.getInstance()``)."""
    _instance = None

    def __init__(self):
        self.codecs = {}
        for c in (NoOp(), Gzip(), Float16(), Int8(), Threshold(), Bitmap()):
            self.codecs[c.NAME] = c
        self.codecs["FTHRESHOLD"] = self.codecs["THRESHOLD"]
        self.default = "FLOAT16"

    @classmethod
    def getInstance(cls):
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def getAvailableCompressors(self): return sorted(self.codecs)
    def getDefaultCompression(self): return self.default

    def setDefaultCompression(self, algorithm):
        if algorithm.upper() not in self.codecs:
            raise ValueError(f"unknown compression algorithm {algorithm}")
        self.default = algorithm.upper()
        return self

    def getCompressor(self, name=None): return self.codecs[(name or self.default).upper()]
    def registerCompressor(self, codec): self.codecs[codec.NAME.upper()] = codec

    def compress(self, arr, algorithm=None): return self.getCompressor(algorithm).compress(arr)
    def compressi(self, arr, algorithm=None): return self.compress(arr, algorithm)

    def decompress(self, c):
        if not isinstance(c, CompressedArray):
            return c
        return self.codecs[c.descriptor.compressionAlgorithm].decompress(c)

    decompressi = decompress
