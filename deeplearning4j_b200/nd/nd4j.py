"""``Nd4j`` static factory (``nd4j-api/.../linalg/factory/Nd4j.java``).

There is no backend SPI: one device model (B200 through torch CUDA, CPU for host-side tests).
``Nd4j.set_default_device`` replaces ``AffinityManager.unsafeSetDevice``.
"""
from __future__ import annotations

import io
import os

import numpy as np
import torch

from .dtype import DataType
from .ndarray import INDArray, NDArrayIndex, _unwrap, wrap


class _Random:
    """``org.nd4j.linalg.api.rng.Random`` over a torch Philox generator per device."""

    def __init__(self):
        self._seed = 0
        self._gens = {}

    def setSeed(self, seed: int):
        self._seed = int(seed)
        self._gens.clear()
        torch.manual_seed(self._seed)

    def getSeed(self):
        return self._seed

    def gen(self, device) -> torch.Generator:
        key = str(device)
        g = self._gens.get(key)
        if g is None:
            g = torch.Generator(device=device)
            g.manual_seed(self._seed)
            self._gens[key] = g
        return g

    def nextDouble(self):
        return float(torch.rand((), generator=self.gen("cpu"), dtype=torch.float64))

    def nextFloat(self):
        return float(torch.rand((), generator=self.gen("cpu")))

    def nextGaussian(self):
        return float(torch.randn((), generator=self.gen("cpu"), dtype=torch.float64))

    def nextInt(self, *a):
        lo, hi = (0, a[0]) if len(a) == 1 else ((a[0], a[1]) if a else (0, 2 ** 31 - 1))
        return int(torch.randint(lo, hi, (), generator=self.gen("cpu")))

    def nextLong(self):
        return self.nextInt(0, 2 ** 62)


class Nd4j:
    EPS_THRESHOLD = 1e-5
    _default_dtype = DataType.FLOAT
    _device = torch.device("cpu")
    _random = _Random()

    # ------------------------------------------------------------------ environment
    @classmethod
    def set_default_device(cls, device):
        cls._device = torch.device(device)

    @classmethod
    def device(cls):
        return cls._device

    @classmethod
    def setDefaultDataTypes(cls, dtype, fp_dtype=None):
        cls._default_dtype = dtype

    @classmethod
    def setDataType(cls, dtype):
        cls._default_dtype = dtype

    @classmethod
    def dataType(cls):
        return cls._default_dtype

    defaultFloatingPointType = dataType

    @classmethod
    def getRandom(cls):
        return cls._random

    @classmethod
    def getExecutioner(cls):
        from ..ops.executioner import OpExecutioner
        return OpExecutioner.instance()

    @classmethod
    def getMemoryManager(cls):
        from ..utils.workspace import MemoryManager
        return MemoryManager.instance()

    @classmethod
    def getWorkspaceManager(cls):
        from ..utils.workspace import WorkspaceManager
        return WorkspaceManager.instance()

    @classmethod
    def getAffinityManager(cls):
        from ..parallel.affinity import AffinityManager
        return AffinityManager.instance()

    @classmethod
    def getCompressor(cls):
        from ..serde.compression import BasicNDArrayCompressor
        return BasicNDArrayCompressor.instance()

    @classmethod
    def getEnvironment(cls):
        from ..utils.environment import Environment
        return Environment.instance()

    # ------------------------------------------------------------------ creation
    @classmethod
    def _td(cls, dtype):
        if dtype is None:
            return cls._default_dtype.to_torch()
        return dtype.to_torch() if isinstance(dtype, DataType) else dtype

    @staticmethod
    def _shape(shape):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
            return tuple(int(s) for s in shape[0])
        return tuple(int(s) for s in shape)

    @classmethod
    def _alloc(cls, fn, shape, dtype, order):
        shape = cls._shape(shape)
        if order == "f" and len(shape) > 1:
            buf = fn(tuple(reversed(shape)), dtype=cls._td(dtype), device=cls._device)
            return INDArray(buf.permute(*reversed(range(len(shape)))), "f")
        return INDArray(fn(shape, dtype=cls._td(dtype), device=cls._device))

    @classmethod
    def create(cls, *args, dtype=None, order="c", shape=None):
        """``Nd4j.create(shape...)``, ``create(data)``, ``create(data, shape)``, ``create(dtype, shape...)``."""
        if args and isinstance(args[0], DataType):
            dtype, args = args[0], args[1:]
        if args and isinstance(args[-1], str) and args[-1] in ("c", "f"):
            order, args = args[-1], args[:-1]
        if not args and shape is not None:
            return cls._alloc(torch.zeros, (shape,), dtype, order)
        first = args[0]
        if isinstance(first, (list, tuple, np.ndarray, torch.Tensor, INDArray)) and not (
                isinstance(first, (list, tuple)) and len(args) == 1 and all(isinstance(v, int) for v in first)
                and shape is None and False):
            is_data = isinstance(first, (np.ndarray, torch.Tensor, INDArray)) or (
                isinstance(first, (list, tuple)) and (len(args) > 1 or shape is not None
                                                      or any(not isinstance(v, int) for v in first)
                                                      or isinstance(first, list)))
            if is_data:
                data = _unwrap(first)
                t = torch.as_tensor(np.asarray(data) if not isinstance(data, torch.Tensor) else data)
                if t.dtype == torch.float64 and dtype is None and not isinstance(data, (np.ndarray, torch.Tensor)):
                    t = t.to(cls._td(None))
                elif dtype is not None:
                    t = t.to(cls._td(dtype))
                t = t.to(cls._device)
                shp = shape if shape is not None else (cls._shape(args[1:]) if len(args) > 1 else None)
                arr = INDArray(t)
                if shp is not None:
                    arr = arr.reshape(*shp, order=order)
                return arr
        return cls._alloc(torch.zeros, args, dtype, order)

    @classmethod
    def createUninitialized(cls, *shape, dtype=None, order="c"):
        if shape and isinstance(shape[0], DataType):
            dtype, shape = shape[0], shape[1:]
        return cls._alloc(torch.empty, shape, dtype, order)

    @classmethod
    def zeros(cls, *shape, dtype=None, order="c"):
        if shape and isinstance(shape[0], DataType):
            dtype, shape = shape[0], shape[1:]
        return cls._alloc(torch.zeros, shape, dtype, order)

    @classmethod
    def ones(cls, *shape, dtype=None, order="c"):
        if shape and isinstance(shape[0], DataType):
            dtype, shape = shape[0], shape[1:]
        return cls._alloc(torch.ones, shape, dtype, order)

    @classmethod
    def valueArrayOf(cls, shape, value, dtype=None):
        shape = cls._shape((shape,)) if isinstance(shape, (tuple, list)) else (int(shape),)
        return INDArray(torch.full(shape, value, dtype=cls._td(dtype), device=cls._device))

    @classmethod
    def scalar(cls, value, dtype=None):
        if dtype is None:
            dtype = (DataType.BOOL if isinstance(value, bool) else DataType.LONG if isinstance(value, int)
                     else cls._default_dtype)
        return INDArray(torch.tensor(value, dtype=cls._td(dtype), device=cls._device))

    @classmethod
    def empty(cls, dtype=None):
        return INDArray(torch.zeros((0,), dtype=cls._td(dtype), device=cls._device))

    @classmethod
    def zerosLike(cls, a): return INDArray(torch.zeros_like(_unwrap(a)))
    @classmethod
    def onesLike(cls, a): return INDArray(torch.ones_like(_unwrap(a)))

    @classmethod
    def eye(cls, n, dtype=None):
        return INDArray(torch.eye(int(n), dtype=cls._td(dtype), device=cls._device))

    @classmethod
    def arange(cls, *a, dtype=None):
        return INDArray(torch.arange(*a, dtype=cls._td(dtype), device=cls._device))

    @classmethod
    def linspace(cls, lo, hi, num, dtype=None):
        return INDArray(torch.linspace(lo, hi, int(num), dtype=cls._td(dtype), device=cls._device))

    @classmethod
    def rand(cls, *shape, dtype=None, seed=None):
        if shape and isinstance(shape[0], DataType):
            dtype, shape = shape[0], shape[1:]
        shape = cls._shape(shape)
        g = cls._random.gen(cls._device) if seed is None else torch.Generator(device=cls._device).manual_seed(seed)
        return INDArray(torch.rand(shape, generator=g, dtype=cls._td(dtype), device=cls._device))

    @classmethod
    def randn(cls, *shape, dtype=None, seed=None):
        if shape and isinstance(shape[0], DataType):
            dtype, shape = shape[0], shape[1:]
        shape = cls._shape(shape)
        g = cls._random.gen(cls._device) if seed is None else torch.Generator(device=cls._device).manual_seed(seed)
        return INDArray(torch.randn(shape, generator=g, dtype=cls._td(dtype), device=cls._device))

    @classmethod
    def randomBernoulli(cls, p, *shape):
        shape = cls._shape(shape)
        g = cls._random.gen(cls._device)
        return INDArray((torch.rand(shape, generator=g, device=cls._device) < p).to(cls._td(None)))

    @classmethod
    def randomExponential(cls, lam, *shape):
        shape = cls._shape(shape)
        g = cls._random.gen(cls._device)
        u = torch.rand(shape, generator=g, device=cls._device, dtype=cls._td(None))
        return INDArray(-torch.log1p(-u) / lam)

    # ------------------------------------------------------------------ combination
    @classmethod
    def concat(cls, dim, *arrs):
        if len(arrs) == 1 and isinstance(arrs[0], (list, tuple)):
            arrs = arrs[0]
        return INDArray(torch.cat([_unwrap(a) for a in arrs], dim=dim))

    @classmethod
    def hstack(cls, *arrs):
        if len(arrs) == 1 and isinstance(arrs[0], (list, tuple)):
            arrs = arrs[0]
        return INDArray(torch.hstack([_unwrap(a) for a in arrs]))

    @classmethod
    def vstack(cls, *arrs):
        if len(arrs) == 1 and isinstance(arrs[0], (list, tuple)):
            arrs = arrs[0]
        return INDArray(torch.vstack([_unwrap(a) for a in arrs]))

    @classmethod
    def stack(cls, dim, *arrs):
        if len(arrs) == 1 and isinstance(arrs[0], (list, tuple)):
            arrs = arrs[0]
        return INDArray(torch.stack([_unwrap(a) for a in arrs], dim=dim))

    @classmethod
    def pile(cls, *arrs):
        return cls.stack(0, *arrs)

    @classmethod
    def tile(cls, a, *reps):
        return INDArray(_unwrap(a).repeat(*reps))

    @classmethod
    def toFlattened(cls, *arrs, order="c"):
        if arrs and isinstance(arrs[0], str):
            order, arrs = arrs[0], arrs[1:]
        if len(arrs) == 1 and isinstance(arrs[0], (list, tuple)):
            arrs = arrs[0]
        return INDArray(torch.cat([wrap(a).ravel(order).t for a in arrs]))

    @classmethod
    def diag(cls, a):
        return INDArray(torch.diag(_unwrap(a).reshape(-1) if _unwrap(a).dim() == 2 and 1 in _unwrap(a).shape else _unwrap(a)))

    @classmethod
    def sort(cls, a, dim=-1, ascending=True):
        return INDArray(torch.sort(_unwrap(a), dim=dim, descending=not ascending).values)

    @classmethod
    def sortWithIndices(cls, a, dim=-1, ascending=True):
        r = torch.sort(_unwrap(a), dim=dim, descending=not ascending)
        return INDArray(r.indices), INDArray(r.values)

    @classmethod
    def argMax(cls, a, *dims):
        return wrap(a).argMax(*dims)

    @classmethod
    def where(cls, cond, x, y):
        return INDArray(torch.where(_unwrap(cond).bool(), _unwrap(x), _unwrap(y)))

    @classmethod
    def gemm(cls, a, b, transposeA=False, transposeB=False, alpha=1.0, beta=0.0, c=None):
        A, B = _unwrap(a), _unwrap(b)
        A = A.t() if transposeA else A
        B = B.t() if transposeB else B
        from ..ops import linalg_dispatch
        out = linalg_dispatch.matmul(A, B) * alpha
        if c is not None:
            C = _unwrap(c)
            C.mul_(beta).add_(out)
            return c
        return INDArray(out)

    @classmethod
    def matmul(cls, a, b, transposeA=False, transposeB=False, transposeResult=False):
        out = cls.gemm(a, b, transposeA, transposeB)
        return out.transpose() if transposeResult else out

    @classmethod
    def tensorMmul(cls, a, b, axes):
        return INDArray(torch.tensordot(_unwrap(a), _unwrap(b), dims=axes))

    @classmethod
    def exec(cls, op, *a, **kw):
        return cls.getExecutioner().exec(op, *a, **kw)

    # ------------------------------------------------------------------ op execution trace (Nd4j.toggleTrace / collectTrace)
    @classmethod
    def toggleTrace(cls, on=True):
        from ..ops import registry
        registry.toggle_trace(on)

    @classmethod
    def purgeTrace(cls):
        from ..ops import registry
        registry.purge_traces()

    @classmethod
    def listTraces(cls):
        from ..ops import registry
        return list(registry.TRACES)

    # ------------------------------------------------------------------ serde
    @classmethod
    def write(cls, arr, out):
        from ..serde.binary import write_array
        write_array(wrap(arr), out)

    @classmethod
    def read(cls, inp):
        from ..serde.binary import read_array
        return read_array(inp, cls._device)

    @classmethod
    def saveBinary(cls, arr, path):
        with open(path, "wb") as f:
            cls.write(arr, f)

    @classmethod
    def readBinary(cls, path):
        with open(path, "rb") as f:
            return cls.read(f)

    @classmethod
    def toByteArray(cls, arr):
        bio = io.BytesIO()
        cls.write(arr, bio)
        return bio.getvalue()

    @classmethod
    def fromByteArray(cls, b):
        return cls.read(io.BytesIO(b))

    @classmethod
    def writeAsNumpy(cls, arr, path):
        np.save(path, wrap(arr).numpy())

    @classmethod
    def createFromNpyFile(cls, path, mmap=False):
        """``mmap=True`` maps the file's data section instead of reading it (host arrays only; writes go back to the file)."""
        if mmap:
            from ..utils.mmap import createFromNpyFileMapped
            return INDArray(createFromNpyFileMapped(path))
        return INDArray(torch.from_numpy(np.load(path)).to(cls._device))

    @classmethod
    def createFromNpzFile(cls, path):
        z = np.load(path)
        return {k: INDArray(torch.from_numpy(z[k]).to(cls._device)) for k in z.files}

    @classmethod
    def toNpyByteArray(cls, arr):
        bio = io.BytesIO()
        np.save(bio, wrap(arr).numpy())
        return bio.getvalue()

    @classmethod
    def createNpyFromByteArray(cls, b):
        return INDArray(torch.from_numpy(np.load(io.BytesIO(b))).to(cls._device))

    @classmethod
    def writeTxt(cls, arr, path):
        a = wrap(arr)
        with open(path, "w") as f:
            f.write(f"{{\n\"filefrom\": \"dl4j\",\n\"ordering\": \"{a.ordering()}\",\n\"shape\":\t{list(a.shape())},\n\"data\":\n")
            f.write(np.array2string(a.numpy(), separator=",", threshold=2 ** 31, max_line_width=10 ** 9))
            f.write("\n}\n")

    @classmethod
    def readTxt(cls, path):
        import ast, re
        s = open(path).read()
        shape = ast.literal_eval(re.search(r'"shape":\s*(\[[^\]]*\])', s).group(1))
        data = s[s.index('"data":') + 7:s.rindex("}")]
        vals = np.array(ast.literal_eval(re.sub(r"\s+", "", data)), dtype=np.float64)
        return INDArray(torch.from_numpy(vals.reshape(shape)).to(cls._td(None)).to(cls._device))


    # ------------------------------------------------------------------ eager op namespaces (NDMath, NDNN, ...)
    @classmethod
    def _ns(cls, name):
        from ..samediff import namespaces as ns
        return getattr(ns, name)(ns.EagerOps())

    @classmethod
    def math(cls): return cls._ns("SDMath")
    @classmethod
    def base(cls): return cls._ns("SDBaseOps")
    @classmethod
    def nn(cls): return cls._ns("SDNN")
    @classmethod
    def cnn(cls): return cls._ns("SDCNN")
    @classmethod
    def rnn(cls): return cls._ns("SDRNN")
    @classmethod
    def loss(cls): return cls._ns("SDLoss")
    @classmethod
    def linalg(cls): return cls._ns("SDLinalg")
    @classmethod
    def image(cls): return cls._ns("SDImage")
    @classmethod
    def bitwise(cls): return cls._ns("SDBitwise")
    @classmethod
    def random(cls): return cls._ns("SDRandom")

    # ------------------------------------------------------------------ reductions over dimensions
    @classmethod
    def _red(cls, fn, a, dims):
        t = _unwrap(a)
        return INDArray(fn(t) if not dims else fn(t, dim=tuple(int(d) for d in dims)))

    @classmethod
    def sum(cls, a, *dims): return cls._red(torch.sum, a, dims)
    @classmethod
    def mean(cls, a, *dims): return cls._red(torch.mean, a, dims)
    @classmethod
    def prod(cls, a, *dims):
        t = _unwrap(a)
        for d in sorted((int(d) % t.dim() for d in dims), reverse=True):
            t = t.prod(d)
        return INDArray(t.prod() if not dims else t)
    @classmethod
    def max(cls, a, *dims): return cls._red(torch.amax, a, dims)
    @classmethod
    def min(cls, a, *dims): return cls._red(torch.amin, a, dims)
    @classmethod
    def std(cls, a, *dims): return cls._red(torch.std, a, dims)
    @classmethod
    def var(cls, a, *dims): return cls._red(torch.var, a, dims)
    @classmethod
    def norm1(cls, a, *dims): return cls._red(lambda t, **k: t.abs().sum(**k), a, dims)
    @classmethod
    def norm2(cls, a, *dims): return cls._red(lambda t, **k: t.pow(2).sum(**k).sqrt(), a, dims)
    @classmethod
    def normmax(cls, a, *dims): return cls._red(lambda t, **k: t.abs().amax(**k) if k else t.abs().max(), a, dims)
    @classmethod
    def cumsum(cls, a, dim=-1): return INDArray(_unwrap(a).cumsum(int(dim)))
    @classmethod
    def argMin(cls, a, *dims):
        t = _unwrap(a)
        return INDArray(t.argmin() if not dims else t.argmin(int(dims[0])))

    # ------------------------------------------------------------------ shape manipulation
    @classmethod
    def append(cls, a, padAmount, val, axis=-1):
        t = _unwrap(a)
        shape = list(t.shape)
        shape[axis] = int(padAmount)
        return INDArray(torch.cat([t, torch.full(shape, val, dtype=t.dtype, device=t.device)], axis))

    @classmethod
    def prepend(cls, a, padAmount, val, axis=-1):
        t = _unwrap(a)
        shape = list(t.shape)
        shape[axis] = int(padAmount)
        return INDArray(torch.cat([torch.full(shape, val, dtype=t.dtype, device=t.device), t], axis))

    @classmethod
    def appendBias(cls, *vectors):
        """Stacks column vectors and appends a 1 (the bias term)."""
        ts = [_unwrap(v).reshape(-1) for v in vectors]
        return INDArray(torch.cat(ts + [torch.ones(1, dtype=ts[0].dtype, device=ts[0].device)]).reshape(-1, 1))

    @classmethod
    def expandDims(cls, a, dim): return INDArray(_unwrap(a).unsqueeze(int(dim)))
    @classmethod
    def squeeze(cls, a, dim): return INDArray(_unwrap(a).squeeze(int(dim)))
    @classmethod
    def stripOnes(cls, a):
        t = _unwrap(a)
        return INDArray(t.reshape([s for s in t.shape if s != 1]))
    @classmethod
    def repeat(cls, a, n): return INDArray(_unwrap(a).reshape(-1).repeat(int(n)))
    @classmethod
    def reverse(cls, a):
        t = _unwrap(a)
        return INDArray(t.reshape(-1).flip(0).reshape(t.shape))
    @classmethod
    def rollAxis(cls, a, axis, start=0): return INDArray(torch.from_numpy(np.rollaxis(wrap(a).numpy(), int(axis), int(start))))
    @classmethod
    def rot90(cls, a): return INDArray(torch.rot90(_unwrap(a), 1, (0, 1)))
    @classmethod
    def pad(cls, a, padWidth, mode="constant", value=0.0):
        t = _unwrap(a)
        pw = np.asarray(_unwrap(padWidth) if not isinstance(padWidth, (list, tuple)) else padWidth).reshape(-1).tolist()
        if len(pw) == 1:
            pw = pw * (2 * t.dim())
        elif len(pw) == 2 and t.dim() > 1:
            pw = pw * t.dim()
        flat = []
        for d in reversed(range(t.dim())):
            flat += [int(pw[2 * d]), int(pw[2 * d + 1])]
        m = {"constant": "constant", "reflect": "reflect", "symmetric": "replicate", "edge": "replicate"}[str(mode).lower()]
        if m == "constant":
            return INDArray(torch.nn.functional.pad(t, flat, value=value))
        return INDArray(torch.nn.functional.pad(t[None], flat, mode=m)[0])
    @classmethod
    def meshgrid(cls, x, y, cartesian=True):
        gx, gy = torch.meshgrid(_unwrap(x).reshape(-1), _unwrap(y).reshape(-1), indexing="xy" if cartesian else "ij")
        return [INDArray(gx), INDArray(gy)]
    @classmethod
    def tri(cls, n, m=None, k=0, dtype=None): return INDArray(torch.tril(torch.ones(int(n), int(m or n), dtype=cls._td(dtype)), int(k)))
    @classmethod
    def triu(cls, a, k=0): return INDArray(torch.triu(_unwrap(a), int(k)))
    @classmethod
    def pullRows(cls, source, sourceDimension, indexes, order="c"):
        """Rows (``sourceDimension`` 1) or columns (0) of ``source`` picked by ``indexes``, stacked along the first axis."""
        t = _unwrap(source)
        idx = torch.as_tensor(list(indexes), dtype=torch.long, device=t.device)
        return INDArray(t.index_select(0, idx) if int(sourceDimension) == 1 else t.index_select(1, idx).t().contiguous())
    @classmethod
    def sortRows(cls, a, columnIdx, ascending=True):
        t = _unwrap(a)
        return INDArray(t[torch.argsort(t[:, int(columnIdx)], descending=not ascending, stable=True)])
    @classmethod
    def sortColumns(cls, a, rowIdx, ascending=True):
        t = _unwrap(a)
        return INDArray(t[:, torch.argsort(t[int(rowIdx)], descending=not ascending, stable=True)])
    @classmethod
    def specialConcat(cls, dim, *arrs): return cls.concat(dim, *arrs)
    @classmethod
    def shuffle(cls, a, *dims, seed=None):
        """In place: permutes the sub-arrays along the given dimension(s) (default: the first)."""
        t = _unwrap(a)
        d = int(dims[0]) if dims else 0
        g = torch.Generator().manual_seed(int(seed)) if seed is not None else cls.getRandom().gen(torch.device("cpu"))
        perm = torch.randperm(t.shape[d], generator=g).to(t.device)
        t.copy_(t.index_select(d, perm))
        return a
    @classmethod
    def clearNans(cls, a):
        t = _unwrap(a)
        t.copy_(torch.nan_to_num(t, nan=0.0))
        return a
    @classmethod
    def copy(cls, a, b): _unwrap(b).copy_(_unwrap(a)); return b
    @classmethod
    def shape(cls, a): return tuple(_unwrap(a).shape)
    @classmethod
    def getStrides(cls, shape, order="c"):
        shape = [int(s) for s in shape]
        st, acc = [0] * len(shape), 1
        rng = range(len(shape)) if order == "f" else reversed(range(len(shape)))
        for i in rng:
            st[i] = acc
            acc *= shape[i]
        return st
    @classmethod
    def order(cls): return "c"
    @classmethod
    def allowsSpecifyOrdering(cls): return True
    @classmethod
    def sizeOfDataType(cls, dtype=None): return torch.empty(0, dtype=cls._td(dtype)).element_size()
    @classmethod
    def emptyWithShape(cls, dtype, *shape): return INDArray(torch.empty(cls._shape(shape), dtype=cls._td(dtype), device=cls._device))
    @classmethod
    def createFromArray(cls, *values):
        v = values[0] if len(values) == 1 else list(values)
        return INDArray(torch.as_tensor(np.asarray(v)).to(cls._device))
    @classmethod
    def createFromFlatArray(cls, flat):
        from ..samediff.serde.flatgraph import from_flat_array
        return INDArray(from_flat_array(flat, cls._device))
    @classmethod
    def choice(cls, source, probs, numSamples, seed=None):
        s, p = _unwrap(source).reshape(-1), _unwrap(probs).reshape(-1).double()
        g = torch.Generator().manual_seed(int(seed)) if seed is not None else cls.getRandom().gen(torch.device("cpu"))
        n = int(numSamples) if not hasattr(numSamples, "shape") else int(np.prod(wrap(numSamples).shape()))
        return INDArray(s[torch.multinomial(p.cpu(), n, replacement=True, generator=g).to(s.device)])
    @classmethod
    def randomBinomial(cls, nTrials, p, *shape):
        g = cls.getRandom().gen(torch.device("cpu"))
        sh = cls._shape(shape)
        return INDArray(torch.binomial(torch.full(sh, float(nTrials)), torch.full(sh, float(p)), generator=g).to(cls._td(None)).to(cls._device))
    @classmethod
    def readNumpy(cls, path, sep=","):
        return INDArray(torch.from_numpy(np.atleast_2d(np.loadtxt(path, delimiter=sep))).to(cls._td(None)).to(cls._device))
    @classmethod
    def readTxtString(cls, stream):
        import tempfile
        data = stream.read() if hasattr(stream, "read") else stream
        with tempfile.NamedTemporaryFile("w", suffix=".txt", delete=False) as f:
            f.write(data.decode() if isinstance(data, bytes) else data)
        try:
            return cls.readTxt(f.name)
        finally:
            import os
            os.unlink(f.name)
    @classmethod
    def convertToNumpy(cls, a): return wrap(a).numpy()
    @classmethod
    def getBackend(cls): return "deeplearning4j_b200 (sm_100a)"
    @classmethod
    def getRandomFactory(cls): return cls.getRandom()
    @classmethod
    def getDistributions(cls):
        from ..nn import weights
        return weights
    @classmethod
    def isExperimentalMode(cls): return False
    @classmethod
    def isFallbackModeEnabled(cls): return False
    @classmethod
    def enableFallbackMode(cls, flag): return None
    @classmethod
    def isPrecisionBoostAllowed(cls): return False
    @classmethod
    def checkShapeValues(cls, *shape):
        for s in cls._shape(shape):
            if s < 0:
                raise ValueError(f"Invalid shape: Requested INDArray shape {list(cls._shape(shape))} contains dimension size values < 0")
    @classmethod
    def close(cls): return None


# ``Transforms`` static helpers (``org.nd4j.linalg.ops.transforms.Transforms``)
class Transforms:
    @staticmethod
    def _u(fn, a, dup=True):
        a = wrap(a)
        if dup:
            return INDArray(fn(a.t))
        a.t.copy_(fn(a.t))
        return a

    sigmoid = staticmethod(lambda a, dup=True: Transforms._u(torch.sigmoid, a, dup))
    tanh = staticmethod(lambda a, dup=True: Transforms._u(torch.tanh, a, dup))
    relu = staticmethod(lambda a, dup=True: Transforms._u(torch.relu, a, dup))
    exp = staticmethod(lambda a, dup=True: Transforms._u(torch.exp, a, dup))
    log = staticmethod(lambda a, dup=True: Transforms._u(torch.log, a, dup))
    sqrt = staticmethod(lambda a, dup=True: Transforms._u(torch.sqrt, a, dup))
    abs = staticmethod(lambda a, dup=True: Transforms._u(torch.abs, a, dup))
    sign = staticmethod(lambda a, dup=True: Transforms._u(torch.sign, a, dup))
    floor = staticmethod(lambda a, dup=True: Transforms._u(torch.floor, a, dup))
    ceil = staticmethod(lambda a, dup=True: Transforms._u(torch.ceil, a, dup))
    round = staticmethod(lambda a, dup=True: Transforms._u(torch.round, a, dup))
    sin = staticmethod(lambda a, dup=True: Transforms._u(torch.sin, a, dup))
    cos = staticmethod(lambda a, dup=True: Transforms._u(torch.cos, a, dup))
    softPlus = staticmethod(lambda a, dup=True: Transforms._u(torch.nn.functional.softplus, a, dup))
    softsign = staticmethod(lambda a, dup=True: Transforms._u(torch.nn.functional.softsign, a, dup))
    hardTanh = staticmethod(lambda a, dup=True: Transforms._u(torch.nn.functional.hardtanh, a, dup))
    elu = staticmethod(lambda a, dup=True: Transforms._u(torch.nn.functional.elu, a, dup))
    neg = staticmethod(lambda a, dup=True: Transforms._u(torch.neg, a, dup))

    @staticmethod
    def leakyRelu(a, alpha=0.01, dup=True):
        return Transforms._u(lambda t: torch.nn.functional.leaky_relu(t, alpha), a, dup)

    @staticmethod
    def pow(a, p, dup=True):
        return Transforms._u(lambda t: torch.pow(t, _unwrap(p)), a, dup)

    @staticmethod
    def softmax(a, dup=True):
        return Transforms._u(lambda t: torch.softmax(t, dim=-1), a, dup)

    @staticmethod
    def max(a, k, dup=True):
        return Transforms._u(lambda t: torch.clamp_min(t, k) if not isinstance(k, INDArray) else torch.maximum(t, k.t), a, dup)

    @staticmethod
    def min(a, k, dup=True):
        return Transforms._u(lambda t: torch.clamp_max(t, k) if not isinstance(k, INDArray) else torch.minimum(t, k.t), a, dup)

    @staticmethod
    def unitVec(a):
        a = wrap(a)
        n = a.t.norm(2)
        return INDArray(a.t / n) if float(n) > 0 else a.dup()

    @staticmethod
    def normalizeZeroMeanAndUnitVariance(a):
        a = wrap(a)
        a.t.sub_(a.t.mean(0, keepdim=True)).div_(a.t.std(0, keepdim=True))
        return a

    @staticmethod
    def cosineSim(a, b):
        a, b = _unwrap(a).reshape(-1).double(), _unwrap(b).reshape(-1).double()
        return float((a @ b) / (a.norm() * b.norm()))

    @staticmethod
    def cosineDistance(a, b):
        return 1.0 - Transforms.cosineSim(a, b)

    @staticmethod
    def euclideanDistance(a, b):
        return float((_unwrap(a).double() - _unwrap(b).double()).norm())

    @staticmethod
    def manhattanDistance(a, b):
        return float((_unwrap(a).double() - _unwrap(b).double()).abs().sum())

    @staticmethod
    def allCosineSimilarities(a, b, *dims):
        A, B = _unwrap(a), _unwrap(b)
        return INDArray(torch.nn.functional.normalize(A, dim=-1) @ torch.nn.functional.normalize(B, dim=-1).t())

    @staticmethod
    def allEuclideanDistances(a, b, *dims):
        return INDArray(torch.cdist(_unwrap(a), _unwrap(b)))

    @staticmethod
    def allManhattanDistances(a, b, *dims):
        return INDArray(torch.cdist(_unwrap(a), _unwrap(b), p=1))
