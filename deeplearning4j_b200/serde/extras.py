"""``org.nd4j.serde``: ``BinarySerde`` (direct byte-buffer round trip), base64 helpers (``Nd4jBase64``), JSON
(de)serialisers for arrays, and the Arrow tensor bridge (``nd4j-serde/nd4j-arrow``; needs ``pyarrow``)."""
from __future__ import annotations

import base64
import io
import json

import numpy as np
import torch

from ..nd.dtype import DataType
from ..nd.ndarray import INDArray
from . import binary


class BinarySerde:
    @staticmethod
    def toByteBuffer(arr) -> bytes: return binary.to_bytes(arr if isinstance(arr, INDArray) else INDArray(arr))
    toArrayAndByteBuffer = toByteBuffer
    @staticmethod
    def toArray(buf) -> INDArray: return binary.from_bytes(bytes(buf))
    @staticmethod
    def writeArrayToDisk(arr, path):
        with open(path, "wb") as f:
            f.write(BinarySerde.toByteBuffer(arr))
    @staticmethod
    def readFromDisk(path):
        with open(path, "rb") as f:
            return BinarySerde.toArray(f.read())
    @staticmethod
    def byteBufferSizeFor(arr): return len(BinarySerde.toByteBuffer(arr))


class Nd4jBase64:
    @staticmethod
    def base64String(arr) -> str: return base64.b64encode(BinarySerde.toByteBuffer(arr)).decode("ascii")
    @staticmethod
    def fromBase64(s) -> INDArray: return BinarySerde.toArray(base64.b64decode(s))
    @staticmethod
    def arraysToBase64(arrs) -> str: return "\t".join(Nd4jBase64.base64String(a) for a in arrs)
    @staticmethod
    def arraysFromBase64(s): return [Nd4jBase64.fromBase64(p) for p in s.split("\t") if p]
    @staticmethod
    def base64StringNumpy(arr) -> str:
        t = arr.t if isinstance(arr, INDArray) else arr
        bio = io.BytesIO()
        np.save(bio, t.detach().cpu().numpy())
        return base64.b64encode(bio.getvalue()).decode("ascii")
    @staticmethod
    def fromNpyBase64(s) -> INDArray: return INDArray(torch.from_numpy(np.load(io.BytesIO(base64.b64decode(s)))))


class NDArrayTextSerializer:
    """JSON form used by ``NDArrayTextSerializer`` / ``NDArrayTextDeSerializer``: dtype, shape, row-major values."""
    @staticmethod
    def toJson(arr) -> str:
        t = (arr.t if isinstance(arr, INDArray) else arr).detach().cpu()
        vals = t.float().reshape(-1).tolist() if t.dtype == torch.bfloat16 else t.reshape(-1).tolist()
        return json.dumps({"dataType": DataType.from_torch(t.dtype).name, "shape": list(t.shape), "data": vals})
    @staticmethod
    def fromJson(s) -> INDArray:
        d = json.loads(s)
        return INDArray(torch.tensor(d["data"], dtype=DataType[d["dataType"]].to_torch()).reshape(d["shape"]))


class ArrowSerde:
    """INDArray <-> Arrow ``Tensor`` (IPC)."""
    @staticmethod
    def toTensor(arr):
        import pyarrow as pa
        t = (arr.t if isinstance(arr, INDArray) else arr).detach().cpu().contiguous()
        return pa.Tensor.from_numpy(t.numpy())
    @staticmethod
    def fromTensor(tensor) -> INDArray: return INDArray(torch.from_numpy(np.array(tensor.to_numpy())))
    @staticmethod
    def toBytes(arr) -> bytes:
        import pyarrow as pa
        sink = pa.BufferOutputStream()
        pa.ipc.write_tensor(ArrowSerde.toTensor(arr), sink)
        return sink.getvalue().to_pybytes()
    @staticmethod
    def fromBytes(b) -> INDArray:
        import pyarrow as pa
        return ArrowSerde.fromTensor(pa.ipc.read_tensor(pa.BufferReader(b)))
