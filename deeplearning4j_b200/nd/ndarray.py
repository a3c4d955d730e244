"""INDArray: the ND4J n-dimensional array surface over a ``torch.Tensor``.

Parity target: ``nd4j-api/.../linalg/api/ndarray/INDArray.java`` (interface) and
``BaseNDArray.java``; native twin ``libnd4j/include/array/NDArray.h:127``.

Design: the array *is* a torch tensor (device-resident on a B200, no host mirror); 'c' / 'f'
ordering is expressed through strides, so an 'f' array is a permuted view of a contiguous buffer
and views share storage exactly as ND4J views do.  In-place methods carry the ND4J ``i`` suffix
(``addi``, ``muli`` ...), copy methods return new arrays.
"""
from __future__ import annotations

from typing import Iterable, Sequence

import numpy as np
import torch

from .dtype import DataType


def _unwrap(x):
    return x.t if isinstance(x, INDArray) else x


def _f_strides(shape):
    st, acc = [], 1
    for s in shape:
        st.append(acc)
        acc *= max(int(s), 1)
    return st


def _c_strides(shape):
    st, acc = [], 1
    for s in reversed(shape):
        st.append(acc)
        acc *= max(int(s), 1)
    return list(reversed(st))


class NDArrayIndex:
    """Index objects mirroring ``org.nd4j.linalg.indexing.NDArrayIndex``."""

    def __init__(self, kind, a=None, b=None, step=1):
        self.kind, self.a, self.b, self.step = kind, a, b, step

    @staticmethod
    def all():
        return NDArrayIndex("all")

    @staticmethod
    def point(i):
        return NDArrayIndex("point", int(i))

    @staticmethod
    def interval(a, b, step=1, inclusive=False):
        if isinstance(step, bool):
            inclusive, step = step, 1
        return NDArrayIndex("interval", int(a), int(b) + (1 if inclusive else 0), int(step))

    @staticmethod
    def indices(*idx):
        return NDArrayIndex("indices", list(idx))

    @staticmethod
    def newAxis():
        return NDArrayIndex("newaxis")

    def to_py(self):
        if self.kind == "all":
            return slice(None)
        if self.kind == "point":
            return self.a
        if self.kind == "interval":
            return slice(self.a, self.b, self.step)
        if self.kind == "indices":
            return list(self.a)
        return None


class INDArray:
    __slots__ = ("t", "_order")
    __array_priority__ = 100

    def __init__(self, t, order: str | None = None):
        if isinstance(t, INDArray):
            t = t.t
        if not isinstance(t, torch.Tensor):
            t = torch.as_tensor(np.asarray(t))
        self.t = t
        self._order = order

    # ------------------------------------------------------------------ meta
    def shape(self):
        return tuple(self.t.shape)

    def size(self, d):
        return self.t.shape[d]

    def rank(self):
        return self.t.dim()

    def length(self):
        return self.t.numel()

    def stride(self):
        return tuple(self.t.stride())

    def rows(self):
        return self.t.shape[0]

    def columns(self):
        return self.t.shape[1] if self.t.dim() > 1 else self.t.shape[0]

    def ordering(self):
        if self._order:
            return self._order
        if self.t.dim() > 1 and not self.t.is_contiguous() and list(self.t.stride()) == _f_strides(self.t.shape):
            return "f"
        return "c"

    def dataType(self):
        return DataType.from_torch(self.t.dtype)

    def isView(self):
        return self.t._base is not None or self.t.storage_offset() != 0

    def isVector(self):
        return self.t.dim() == 1 or (self.t.dim() == 2 and min(self.t.shape) == 1)

    def isRowVector(self):
        return self.t.dim() == 1 or (self.t.dim() == 2 and self.t.shape[0] == 1)

    def isColumnVector(self):
        return self.t.dim() == 2 and self.t.shape[1] == 1

    def isMatrix(self):
        return self.t.dim() == 2

    def isScalar(self):
        return self.t.numel() == 1

    def isEmpty(self):
        return self.t.numel() == 0

    def isR(self):
        return self.t.dtype.is_floating_point

    def isZ(self):
        return not self.t.dtype.is_floating_point and self.t.dtype != torch.bool

    def isB(self):
        return self.t.dtype == torch.bool

    def device(self):
        return self.t.device

    def elementWiseStride(self):
        if self.t.is_contiguous():
            return 1
        if list(self.t.stride()) == _f_strides(self.t.shape):
            return 1
        return 0

    def shapeInfo(self):
        """ND4J shape-info longs ``[rank, shape.., stride.., extras, ews, order]``."""
        from .dtype import extras_for
        sh = list(self.t.shape)
        order = self.ordering()
        st = _f_strides(sh) if order == "f" else _c_strides(sh)
        return [len(sh)] + sh + st + [extras_for(self.dataType(), self.t.numel() == 0), 1, ord(order)]

    # ------------------------------------------------------------------ conversion
    def toTorch(self):
        return self.t

    def numpy(self):
        t = self.t.detach().cpu()
        if t.dtype == torch.bfloat16:
            t = t.float()
        return t.numpy()

    def toDoubleVector(self):
        return self.t.detach().double().cpu().reshape(-1).tolist()

    def toFloatVector(self):
        return self.t.detach().float().cpu().reshape(-1).tolist()

    def toIntVector(self):
        return self.t.detach().to(torch.int64).cpu().reshape(-1).tolist()

    toLongVector = toIntVector

    def toDoubleMatrix(self):
        return self.t.detach().double().cpu().tolist()

    toFloatMatrix = toDoubleMatrix

    def getDouble(self, *idx):
        if len(idx) == 1 and self.t.dim() != 1:
            return float(self.ravel().t[idx[0]])
        return float(self.t[tuple(idx)])

    getFloat = getDouble

    def getInt(self, *idx):
        return int(self.getDouble(*idx))

    getLong = getInt

    def getScalar(self, *idx):
        return INDArray(self.t[tuple(idx)].reshape(()))

    def sumNumber(self):
        return float(self.t.sum())

    def meanNumber(self):
        return float(self.t.float().mean()) if not self.t.dtype.is_floating_point else float(self.t.mean())

    def maxNumber(self):
        return float(self.t.max())

    def minNumber(self):
        return float(self.t.min())

    def stdNumber(self, biasCorrected=True):
        return float(self.t.std(unbiased=biasCorrected))

    def varNumber(self, biasCorrected=True):
        return float(self.t.var(unbiased=biasCorrected))

    def norm1Number(self):
        return float(self.t.abs().sum())

    def norm2Number(self):
        return float(self.t.float().norm(2))

    def normmaxNumber(self):
        return float(self.t.abs().max())

    def prodNumber(self):
        return float(self.t.prod())

    def castTo(self, dtype):
        dt = dtype.to_torch() if isinstance(dtype, DataType) else dtype
        return INDArray(self.t.to(dt))

    def to(self, device):
        return INDArray(self.t.to(device), self._order)

    # ------------------------------------------------------------------ copy / views
    def dup(self, order: str | None = None):
        order = order or self.ordering()
        if order == "f" and self.t.dim() > 1:
            nd = self.t.dim()
            buf = self.t.permute(*reversed(range(nd))).contiguous()
            return INDArray(buf.permute(*reversed(range(nd))), "f")
        return INDArray(self.t.contiguous().clone(), "c")

    def detach(self):
        return INDArray(self.t.detach(), self._order)

    def assign(self, other):
        o = _unwrap(other)
        if isinstance(o, torch.Tensor):
            self.t.copy_(o.to(self.t.dtype).expand_as(self.t) if o.shape != self.t.shape and o.numel() != self.t.numel()
                         else o.reshape(self.t.shape).to(self.t.dtype))
        else:
            self.t.fill_(o)
        return self

    def ravel(self, order: str = "c"):
        if order == "f" and self.t.dim() > 1:
            nd = self.t.dim()
            return INDArray(self.t.permute(*reversed(range(nd))).reshape(-1))
        return INDArray(self.t.reshape(-1))

    def reshape(self, *shape, order: str | None = None):
        if len(shape) and isinstance(shape[0], str):
            order, shape = shape[0], shape[1:]
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        order = order or "c"
        if order == "f":
            nd = self.t.dim()
            flat = self.t.permute(*reversed(range(nd))).reshape(-1) if nd > 1 else self.t.reshape(-1)
            out = flat.reshape(tuple(reversed(shape)))
            return INDArray(out.permute(*reversed(range(len(shape)))), "f")
        return INDArray(self.t.reshape(shape))

    def permute(self, *dims):
        if len(dims) == 1 and isinstance(dims[0], (tuple, list)):
            dims = tuple(dims[0])
        return INDArray(self.t.permute(*dims))

    def transpose(self):
        if self.t.dim() < 2:
            return INDArray(self.t.reshape(-1, 1) if self.t.dim() == 1 else self.t)
        return INDArray(self.t.transpose(-1, -2) if self.t.dim() == 2 else self.t.permute(*reversed(range(self.t.dim()))))

    def swapAxes(self, a, b):
        return INDArray(self.t.transpose(a, b))

    def broadcast(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        return INDArray(self.t.expand(*shape))

    def repmat(self, *reps):
        return INDArray(self.t.repeat(*reps))

    def repeat(self, dim, *reps):
        return INDArray(torch.repeat_interleave(self.t, reps[0], dim=dim))

    def get(self, *indexes):
        py, newaxes = [], []
        for k, ix in enumerate(indexes):
            if isinstance(ix, NDArrayIndex):
                if ix.kind == "newaxis":
                    py.append(None)
                elif ix.kind == "point":
                    py.append(ix.a)
                else:
                    py.append(ix.to_py())
            else:
                py.append(ix)
        return INDArray(self.t[tuple(py)])

    def put(self, indexes, value=None):
        if value is None:
            raise ValueError("put(indexes, value)")
        if isinstance(indexes, (list, tuple)) and len(indexes) and isinstance(indexes[0], NDArrayIndex):
            py = tuple(ix.to_py() for ix in indexes)
        else:
            py = indexes
        v = _unwrap(value)
        self.t[py] = v if not isinstance(v, torch.Tensor) else v.to(self.t.dtype)
        return self

    def putScalar(self, *args):
        *idx, v = args
        if len(idx) == 1 and isinstance(idx[0], (list, tuple)):
            idx = list(idx[0])
        if len(idx) == 1 and self.t.dim() != 1:
            self.t.view(-1)[idx[0]] = v
        else:
            self.t[tuple(idx)] = v
        return self

    def getRow(self, i, keepDim=False):
        r = self.t[i]
        return INDArray(r.unsqueeze(0) if keepDim else r)

    def getColumn(self, i, keepDim=False):
        r = self.t[:, i]
        return INDArray(r.unsqueeze(1) if keepDim else r)

    def getRows(self, *rows):
        return INDArray(self.t[list(rows)])

    def getColumns(self, *cols):
        return INDArray(self.t[:, list(cols)])

    def putRow(self, i, row):
        self.t[i] = _unwrap(row).reshape(self.t[i].shape)
        return self

    def putColumn(self, i, col):
        self.t[:, i] = _unwrap(col).reshape(self.t[:, i].shape)
        return self

    def slice(self, i, dim=0):
        return INDArray(self.t.select(dim, i))

    def tensorAlongDimension(self, index, *dims):
        nd = self.t.dim()
        dims = [d % nd for d in dims]
        other = [d for d in range(nd) if d not in dims]
        perm = other + dims
        p = self.t.permute(*perm)
        lead = int(np.prod([self.t.shape[d] for d in other])) if other else 1
        p = p.reshape((lead,) + tuple(self.t.shape[d] for d in dims))
        return INDArray(p[index])

    def tensorsAlongDimension(self, *dims):
        nd = self.t.dim()
        dims = [d % nd for d in dims]
        return int(np.prod([self.t.shape[d] for d in range(nd) if d not in dims]))

    def vectorAlongDimension(self, index, dim):
        return self.tensorAlongDimension(index, dim)

    def __getitem__(self, item):
        if isinstance(item, tuple):
            item = tuple(_unwrap(i) for i in item)
        else:
            item = _unwrap(item)
        return INDArray(self.t[item])

    def __setitem__(self, item, value):
        self.t[item] = _unwrap(value)

    def __len__(self):
        return self.t.shape[0]

    # ------------------------------------------------------------------ arithmetic
    def _bin(self, other, fn):
        return INDArray(fn(self.t, _unwrap(other)))

    def _ibin(self, other, fn):
        fn(self.t, _unwrap(other))
        return self

    def add(self, o): return self._bin(o, torch.add)
    def sub(self, o): return self._bin(o, torch.sub)
    def mul(self, o): return self._bin(o, torch.mul)
    def div(self, o): return self._bin(o, torch.div)
    def rsub(self, o): return INDArray(_unwrap(o) - self.t)
    def rdiv(self, o): return INDArray(_unwrap(o) / self.t)
    def addi(self, o): self.t.add_(_unwrap(o)); return self
    def subi(self, o): self.t.sub_(_unwrap(o)); return self
    def muli(self, o): self.t.mul_(_unwrap(o)); return self
    def divi(self, o): self.t.div_(_unwrap(o)); return self
    def rsubi(self, o): self.t.copy_(_unwrap(o) - self.t); return self
    def rdivi(self, o): self.t.copy_(_unwrap(o) / self.t); return self
    def neg(self): return INDArray(-self.t)
    def negi(self): self.t.neg_(); return self
    def fmod(self, o): return self._bin(o, torch.fmod)
    def remainder(self, o): return self._bin(o, torch.remainder)

    __add__ = add
    __sub__ = sub
    __mul__ = mul
    __truediv__ = div
    __radd__ = add
    __rmul__ = mul
    def __rsub__(self, o): return self.rsub(o)
    def __rtruediv__(self, o): return self.rdiv(o)
    def __neg__(self): return self.neg()
    def __matmul__(self, o): return self.mmul(o)

    # row/column vector broadcasts
    def _rowop(self, v, fn, inplace):
        v = _unwrap(v).reshape(1, -1)
        if inplace:
            fn(self.t, v, out=self.t)
            return self
        return INDArray(fn(self.t, v))

    def _colop(self, v, fn, inplace):
        v = _unwrap(v).reshape(-1, 1)
        if inplace:
            fn(self.t, v, out=self.t)
            return self
        return INDArray(fn(self.t, v))

    def addRowVector(self, v): return self._rowop(v, torch.add, False)
    def addiRowVector(self, v): return self._rowop(v, torch.add, True)
    def subRowVector(self, v): return self._rowop(v, torch.sub, False)
    def subiRowVector(self, v): return self._rowop(v, torch.sub, True)
    def mulRowVector(self, v): return self._rowop(v, torch.mul, False)
    def muliRowVector(self, v): return self._rowop(v, torch.mul, True)
    def divRowVector(self, v): return self._rowop(v, torch.div, False)
    def diviRowVector(self, v): return self._rowop(v, torch.div, True)
    def addColumnVector(self, v): return self._colop(v, torch.add, False)
    def addiColumnVector(self, v): return self._colop(v, torch.add, True)
    def subColumnVector(self, v): return self._colop(v, torch.sub, False)
    def subiColumnVector(self, v): return self._colop(v, torch.sub, True)
    def mulColumnVector(self, v): return self._colop(v, torch.mul, False)
    def muliColumnVector(self, v): return self._colop(v, torch.mul, True)
    def divColumnVector(self, v): return self._colop(v, torch.div, False)
    def diviColumnVector(self, v): return self._colop(v, torch.div, True)

    # linear algebra
    def mmul(self, other, result=None):
        from ..ops import linalg_dispatch
        out = linalg_dispatch.matmul(self.t, _unwrap(other))
        if result is not None:
            _unwrap(result).copy_(out)
            return result
        return INDArray(out)

    def mmuli(self, other):
        return self.assign(self.mmul(other))

    def dot(self, other):
        return float((self.t.reshape(-1) * _unwrap(other).reshape(-1)).sum())

    # comparisons -> BOOL arrays
    def gt(self, o): return self._bin(o, torch.gt)
    def gte(self, o): return self._bin(o, torch.ge)
    def lt(self, o): return self._bin(o, torch.lt)
    def lte(self, o): return self._bin(o, torch.le)
    def eq(self, o): return self._bin(o, torch.eq)
    def neq(self, o): return self._bin(o, torch.ne)
    def isNaN(self): return INDArray(torch.isnan(self.t))
    def isInfinite(self): return INDArray(torch.isinf(self.t))
    def any(self): return bool(self.t.any())
    def all(self): return bool(self.t.all())
    def none(self): return not bool(self.t.any())

    def equalsWithEps(self, other, eps=1e-5):
        o = _unwrap(other)
        if tuple(o.shape) != tuple(self.t.shape):
            return False
        if self.t.numel() == 0:
            return True
        return bool((self.t.double() - o.to(self.t.device).double()).abs().max() <= eps)

    def equals(self, other):
        return isinstance(other, INDArray) and self.equalsWithEps(other, 1e-5)

    def equalShapes(self, other):
        return tuple(self.t.shape) == tuple(_unwrap(other).shape)

    __eq__ = None  # set below

    # reductions
    def _red(self, fn, dims, keepDims=False, **kw):
        if len(dims) == 1 and isinstance(dims[0], (tuple, list)):
            dims = tuple(dims[0])
        if len(dims) and isinstance(dims[0], bool):
            keepDims, dims = dims[0], dims[1:]
        if not dims:
            return INDArray(fn(self.t, **kw)) if not kw else INDArray(fn(self.t, dim=None, **kw))
        return INDArray(fn(self.t, dim=tuple(dims), keepdim=keepDims, **kw))

    def sum(self, *dims, keepDims=False): return self._red(torch.sum, dims, keepDims)
    def mean(self, *dims, keepDims=False): return self._red(torch.mean, dims, keepDims)
    def prod(self, *dims, keepDims=False):
        if not dims:
            return INDArray(self.t.prod())
        t = self.t
        for d in sorted([d % t.dim() for d in dims], reverse=True):
            t = t.prod(dim=d, keepdim=keepDims)
        return INDArray(t)
    def max(self, *dims, keepDims=False): return self._red(torch.amax, dims, keepDims)
    def min(self, *dims, keepDims=False): return self._red(torch.amin, dims, keepDims)
    def amax(self, *dims): return INDArray(self.t.abs())._red(torch.amax, dims)
    def amin(self, *dims): return INDArray(self.t.abs())._red(torch.amin, dims)
    def amean(self, *dims): return INDArray(self.t.abs())._red(torch.mean, dims)
    def std(self, *dims, biasCorrected=True):
        if dims and isinstance(dims[0], bool):
            biasCorrected, dims = dims[0], dims[1:]
        return INDArray(self.t.std(dim=tuple(dims) if dims else None, unbiased=biasCorrected))
    def var(self, *dims, biasCorrected=True):
        if dims and isinstance(dims[0], bool):
            biasCorrected, dims = dims[0], dims[1:]
        return INDArray(self.t.var(dim=tuple(dims) if dims else None, unbiased=biasCorrected))
    def norm1(self, *dims): return INDArray(self.t.abs())._red(torch.sum, dims)
    def norm2(self, *dims): return INDArray((self.t * self.t))._red(torch.sum, dims)._sqrt()
    def normmax(self, *dims): return INDArray(self.t.abs())._red(torch.amax, dims)
    def _sqrt(self): return INDArray(self.t.sqrt())
    def argMax(self, *dims):
        if not dims:
            return INDArray(self.t.argmax())
        return INDArray(self.t.argmax(dim=dims[0]))
    def argMin(self, *dims):
        if not dims:
            return INDArray(self.t.argmin())
        return INDArray(self.t.argmin(dim=dims[0]))
    def cumsum(self, dim): return INDArray(self.t.cumsum(dim))
    def cumsumi(self, dim): self.t.copy_(self.t.cumsum(dim)); return self
    def entropy(self, *dims): return INDArray(-(self.t * self.t.log()))._red(torch.sum, dims)
    def logEntropy(self, *dims): return INDArray(self.entropy(*dims).t.log())
    def shannonEntropy(self, *dims): return INDArray(-(self.t * self.t.log2()))._red(torch.sum, dims)

    def distance1(self, o): return float((self.t - _unwrap(o)).abs().sum())
    def distance2(self, o): return float((self.t - _unwrap(o)).norm(2))
    def squaredDistance(self, o): return float(((self.t - _unwrap(o)) ** 2).sum())

    # misc
    def like(self): return INDArray(torch.zeros_like(self.t))
    def ulike(self): return INDArray(torch.empty_like(self.t))
    def isAttached(self): return False
    def close(self): return None
    def closeable(self): return True
    def wasClosed(self): return False
    def leverageTo(self, _id, *a): return self
    def migrate(self, *a): return self
    def detachFromWorkspace(self): return self
    def data(self): return self.t.reshape(-1) if self.t.is_contiguous() else self.t.contiguous().reshape(-1)

    # ------------------------------------------------------------------ reverse row / column vector ops, fmod / remainder in place
    def rsubRowVector(self, v): return INDArray(_unwrap(v).reshape(1, -1) - self.t)
    def rsubiRowVector(self, v): self.t.copy_(_unwrap(v).reshape(1, -1) - self.t); return self
    def rdivRowVector(self, v): return INDArray(_unwrap(v).reshape(1, -1) / self.t)
    def rdiviRowVector(self, v): self.t.copy_(_unwrap(v).reshape(1, -1) / self.t); return self
    def rsubColumnVector(self, v): return INDArray(_unwrap(v).reshape(-1, 1) - self.t)
    def rsubiColumnVector(self, v): self.t.copy_(_unwrap(v).reshape(-1, 1) - self.t); return self
    def rdivColumnVector(self, v): return INDArray(_unwrap(v).reshape(-1, 1) / self.t)
    def rdiviColumnVector(self, v): self.t.copy_(_unwrap(v).reshape(-1, 1) / self.t); return self
    def putiRowVector(self, v): self.t.copy_(_unwrap(v).reshape(1, -1).expand_as(self.t)); return self
    def putiColumnVector(self, v): self.t.copy_(_unwrap(v).reshape(-1, 1).expand_as(self.t)); return self
    def fmodi(self, o): self.t.fmod_(_unwrap(o)); return self
    def remainderi(self, o): self.t.remainder_(_unwrap(o)); return self

    # ------------------------------------------------------------------ conditions (Conditions / BooleanIndexing)
    def cond(self, condition):
        """1 where the condition holds, 0 elsewhere (a new array of this array's type)."""
        return INDArray(condition.apply(self.t).to(self.t.dtype))

    def match(self, comp, condition):
        """Boolean array: the condition evaluated with ``comp`` (a number or an array) as the comparison value."""
        from .conditions import Condition
        c = Condition(condition.mode, _unwrap(comp), condition._fn, condition.name)
        return INDArray(c.apply(self.t))

    def getWhere(self, comp, condition):
        """The elements that satisfy the condition against ``comp``, as a vector."""
        return INDArray(self.t[self.match(comp, condition).t])

    def putWhere(self, comp, put, condition):
        """A copy in which the elements that satisfy the condition against ``comp`` are replaced by ``put``."""
        m = self.match(comp, condition).t
        out, p = self.t.clone(), _unwrap(put)
        if isinstance(p, torch.Tensor) and p.numel() > 1:
            out[m] = p.to(out.dtype).expand_as(out)[m]
        else:
            out[m] = float(p)
        return INDArray(out)

    def putWhereWithMask(self, mask, put):
        m = _unwrap(mask).bool()
        out, p = self.t.clone(), _unwrap(put)
        if isinstance(p, torch.Tensor) and p.numel() > 1:
            out[m] = p.to(out.dtype).expand_as(out)[m]
        else:
            out[m] = float(p)
        return INDArray(out)

    def replaceWhere(self, arr, condition):
        """In place: elements that satisfy the condition are taken from ``arr``."""
        m = condition.apply(self.t)
        self.t[m] = _unwrap(arr).to(self.t.dtype).expand_as(self.t)[m]
        return self

    def assignIf(self, arr, condition):
        """In place: elements of ``arr`` that satisfy the condition are copied into this array."""
        a = _unwrap(arr).to(self.t.dtype).expand_as(self.t)
        m = condition.apply(a)
        self.t[m] = a[m]
        return self

    def scan(self, condition):
        """Number of elements that satisfy the condition."""
        return int(condition.apply(self.t).sum())

    def eps(self, o):
        o = _unwrap(o)
        return INDArray((self.t - o).abs() < 1e-5)

    # ------------------------------------------------------------------ order statistics and entropies
    def percentileNumber(self, q):
        """Linear-interpolated percentile (``q`` in [0, 100]) over all elements, as the reference computes it on the sorted copy:
        position q / 100 * (n + 1) - 1 clamped to the ends."""
        v = self.t.reshape(-1).double().sort().values
        n = v.numel()
        if q <= 0:
            return float(v[0])
        if q >= 100:
            return float(v[-1])
        pos = q / 100.0 * (n + 1)
        if pos < 1:
            return float(v[0])
        if pos >= n:
            return float(v[-1])
        lo = int(pos)
        return float(v[lo - 1] + (pos - lo) * (v[lo] - v[lo - 1]))

    def medianNumber(self): return self.percentileNumber(50)

    def percentile(self, q, *dims):
        if not dims:
            return INDArray(torch.tensor(self.percentileNumber(q), dtype=self.t.dtype))
        dims = sorted(d % self.t.dim() for d in dims)
        keep = [d for d in range(self.t.dim()) if d not in dims]
        flat = self.t.permute(*keep, *dims).reshape(*[self.t.shape[d] for d in keep], -1)
        out = torch.empty(flat.shape[:-1], dtype=self.t.dtype)
        for i in range(out.numel()):
            out.reshape(-1)[i] = INDArray(flat.reshape(-1, flat.shape[-1])[i]).percentileNumber(q)
        return INDArray(out)

    def median(self, *dims): return self.percentile(50, *dims)
    def amaxNumber(self): return float(self.t.abs().max())
    def aminNumber(self): return float(self.t.abs().min())
    def ameanNumber(self): return float(self.t.abs().double().mean())

    def entropyNumber(self):
        x = self.t.double()
        return float(-(x * torch.log(x)).sum())

    def shannonEntropyNumber(self):
        x = self.t.double()
        return float(-(x * torch.log2(x)).sum())

    def logEntropyNumber(self):
        import math
        return math.log(self.entropyNumber())

    # ------------------------------------------------------------------ shape queries, in-place permutes, slices
    def isSquare(self): return self.t.dim() == 2 and self.t.shape[0] == self.t.shape[1]
    def isVectorOrScalar(self): return self.isVector() or self.t.numel() == 1
    def isRowVectorOrScalar(self): return self.isRowVector() or self.t.numel() == 1
    def isColumnVectorOrScalar(self): return self.isColumnVector() or self.t.numel() == 1
    def isSparse(self): return False
    def isCompressed(self): return False
    def isS(self): return False
    def isInScope(self): return True
    def getWorkspace(self): return None
    def markAsCompressed(self, flag): return None
    def setCloseable(self, flag): return None
    def offset(self): return int(self.t.storage_offset())
    def originalOffset(self): return int(self.t.storage_offset())
    def getId(self): return id(self)
    def element(self): return self.t.reshape(-1)[0].item()
    def getNumber(self, *idx): return self.t[tuple(int(i) for i in idx)].item() if idx else self.element()
    def getDoubleUnsafe(self, offset): return float(self.data()[int(offset)])

    def putScalarUnsafe(self, offset, value):
        self.t.reshape(-1)[int(offset)] = value
        return self

    def getLeadingOnes(self):
        n = 0
        for s in self.t.shape:
            if s != 1:
                break
            n += 1
        return n

    def getTrailingOnes(self):
        n = 0
        for s in reversed(self.t.shape):
            if s != 1:
                break
            n += 1
        return n

    def permutei(self, *dims):
        if len(dims) == 1 and isinstance(dims[0], (tuple, list)):
            dims = tuple(dims[0])
        self.t = self.t.permute(*dims)
        self._order = None
        return self

    def transposei(self):
        self.t = self.t.t() if self.t.dim() == 2 else self.t.permute(*reversed(range(self.t.dim())))
        self._order = None
        return self

    def dimShuffle(self, rearrange, newOrder=None, broadCastable=None):
        """Permute with ``'x'`` entries inserting broadcastable axes of length 1."""
        perm = [r for r in rearrange if r != "x"]
        t = self.t.permute(*[int(p) for p in perm])
        for i, r in enumerate(rearrange):
            if r == "x":
                t = t.unsqueeze(i)
        return INDArray(t)

    def slices(self): return self.t.shape[0]
    def putSlice(self, i, arr): self.t[int(i)] = _unwrap(arr); return self
    def vectorsAlongDimension(self, dim): return self.t.numel() // self.t.shape[dim] if self.t.numel() else 0

    def sliceVectors(self, out=None):
        out = [] if out is None else out
        if self.t.dim() <= 1:
            out.append(self)
        else:
            for i in range(self.t.shape[0]):
                INDArray(self.t[i]).sliceVectors(out)
        return out

    def setOrder(self, order): self._order = str(order); return self
    def setData(self, data): self.t.reshape(-1).copy_(_unwrap(data).reshape(-1)); return self

    def setShapeAndStride(self, shape, stride):
        self.t = self.t.as_strided(tuple(int(s) for s in shape), tuple(int(s) for s in stride), self.t.storage_offset())
        return self

    def unsafeDuplication(self, blocking=True): return INDArray(self.t.clone())
    def leverage(self): return self
    def leverageOrDetach(self, _id): return self
    def toFlatArray(self, builder=None):
        from ..samediff.serde.flatgraph import flat_array
        return flat_array(self.t)

    def toIntMatrix(self): return self.t.to(torch.int32).reshape(self.t.shape[0], -1).tolist()
    def toLongMatrix(self): return self.t.to(torch.int64).reshape(self.t.shape[0], -1).tolist()
    def getString(self, index): raise TypeError("getString applies to UTF8 arrays; this array holds " + self.dataType().name)

    # ------------------------------------------------------------------ shape descriptors and text
    def shapeInfoJava(self):
        """[rank, shape..., stride..., type flags, element-wise stride, order char]: the shapeInfo vector of the reference."""
        st = list(self.t.stride())
        ews = 1 if self.t.is_contiguous() else 0
        return [self.t.dim(), *self.t.shape, *st, 0, ews, ord(self.ordering())]

    def shapeInfoDataBuffer(self): return torch.tensor(self.shapeInfoJava(), dtype=torch.int64)
    def shapeDescriptor(self):
        return {"shape": tuple(self.t.shape), "stride": tuple(self.t.stride()), "order": self.ordering(), "dataType": self.dataType(),
                "offset": self.offset(), "ews": 1 if self.t.is_contiguous() else 0}

    def shapeInfoToString(self):
        return (f"Rank: {self.t.dim()}, DataType: {self.dataType().name}, Offset: {self.offset()}, Order: {self.ordering()}, "
                f"Shape: {list(self.t.shape)}, Stride: {list(self.t.stride())}")

    def toString(self, *a, **kw): return repr(self.t.tolist())
    def toStringFull(self):
        with torch._tensor_str.printoptions(threshold=1 << 62):
            return str(self.t)

    # event / allocation tracing of the reference's debug builds: nothing is recorded here
    def addEvent(self, event): return None
    def writeEvents(self, *a): return []
    def allocationTrace(self): return None
    def getOrCreateOpaqueNDArray(self): return self
    def clearOpaqueNDArray(self): return None
    def log(self, *a): return None

    def __repr__(self):
        return f"INDArray(shape={list(self.t.shape)}, dtype={self.dataType().name}, order='{self.ordering()}')\n{self.t}"

    def __array__(self, dtype=None):
        a = self.numpy()
        return a.astype(dtype) if dtype is not None else a

    def __hash__(self):
        return id(self)


def _eq(self, other):
    if isinstance(other, INDArray):
        return self.equals(other)
    return NotImplemented


INDArray.__eq__ = _eq


def wrap(x) -> INDArray:
    return x if isinstance(x, INDArray) else INDArray(x)
