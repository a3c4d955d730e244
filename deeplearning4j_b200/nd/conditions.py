"""``Conditions`` and ``BooleanIndexing`` (``nd4j-api/.../linalg/indexing/conditions/Conditions.java``, ``BooleanIndexing.java``):
element-wise predicates with the reference's mode numbers, composable with ``And`` / ``Or`` / ``Not``, and the masked
assignment helpers built on them."""
from __future__ import annotations

import torch

_EPS = 1e-5


class Condition:
    """A predicate over array elements.  ``mode`` is the reference's ``ConditionMode`` number (-1 for aggregates)."""

    def __init__(self, mode, value=0.0, fn=None, name=""):
        self.mode, self.value, self._fn, self.name = int(mode), value, fn, name

    def apply(self, t: torch.Tensor) -> torch.Tensor:
        return self._fn(t, self.value)

    def __call__(self, x):
        from .ndarray import INDArray
        t = x.t if isinstance(x, INDArray) else torch.as_tensor(x)
        return self.apply(t)

    def condtionNum(self):          # (sic) the reference's spelling
        return self.mode

    conditionNum = condtionNum

    def getValue(self):
        return self.value

    def __repr__(self):
        return f"Condition({self.name}, {self.value})"


def _mk(mode, name, fn):
    def make(value=0.0):
        return Condition(mode, value, fn, name)
    make.__name__ = name
    return staticmethod(make)


class Conditions:
    epsEquals = _mk(0, "epsEquals", lambda x, c: (x - c).abs() <= _EPS)
    epsNotEquals = _mk(1, "epsNotEquals", lambda x, c: (x - c).abs() > _EPS)
    lessThan = _mk(2, "lessThan", lambda x, c: x < c)
    greaterThan = _mk(3, "greaterThan", lambda x, c: x > c)
    lessThanOrEqual = _mk(4, "lessThanOrEqual", lambda x, c: x <= c)
    greaterThanOrEqual = _mk(5, "greaterThanOrEqual", lambda x, c: x >= c)
    absLessThan = _mk(6, "absLessThan", lambda x, c: x.abs() < c)
    absGreaterThan = _mk(7, "absGreaterThan", lambda x, c: x.abs() > c)
    isInfinite = _mk(8, "isInfinite", lambda x, c: torch.isinf(x))
    isNan = _mk(9, "isNan", lambda x, c: torch.isnan(x))
    equals = _mk(10, "equals", lambda x, c: x == c)
    notEquals = _mk(11, "notEquals", lambda x, c: x != c)
    absGreaterThanOrEqual = _mk(12, "absGreaterThanOrEqual", lambda x, c: x.abs() >= c)
    absLessThanOrEqual = _mk(13, "absLessThanOrEqual", lambda x, c: x.abs() <= c)
    isFinite = _mk(14, "isFinite", lambda x, c: torch.isfinite(x))
    notFinite = _mk(15, "notFinite", lambda x, c: ~torch.isfinite(x))

    @staticmethod
    def fromInt(mode, value=0.0):
        for n in dir(Conditions):
            f = getattr(Conditions, n)
            if callable(f) and n not in ("fromInt",) and not n.startswith("_"):
                c = f(value)
                if isinstance(c, Condition) and c.mode == int(mode):
                    return c
        raise ValueError(f"unknown condition mode {mode}")


def And(*conds):
    return Condition(-1, None, lambda x, _: torch.stack([c.apply(x) for c in conds]).all(0), "and")


def Or(*conds):
    return Condition(-1, None, lambda x, _: torch.stack([c.apply(x) for c in conds]).any(0), "or")


def Not(cond):
    return Condition(-1, None, lambda x, _: ~cond.apply(x), "not")


class BooleanIndexing:
    @staticmethod
    def _t(x):
        from .ndarray import INDArray
        return x.t if isinstance(x, INDArray) else x

    @staticmethod
    def and_(arr, cond):
        return bool(cond.apply(BooleanIndexing._t(arr)).all())

    @staticmethod
    def or_(arr, cond):
        return bool(cond.apply(BooleanIndexing._t(arr)).any())

    @staticmethod
    def replaceWhere(to, put, cond):
        """In place: elements of ``to`` that satisfy ``cond`` become ``put`` (a number, or an array of the same shape)."""
        t = BooleanIndexing._t(to)
        m = cond.apply(t)
        p = BooleanIndexing._t(put)
        if isinstance(p, torch.Tensor) and p.numel() > 1:
            t[m] = p.to(t.dtype)[m]
        else:
            t[m] = float(p) if not isinstance(p, torch.Tensor) else p.to(t.dtype).reshape(())
        return to

    @staticmethod
    def chooseFrom(arrs, cond=None, scalars=None):
        from .ndarray import INDArray
        t = BooleanIndexing._t(arrs[0])
        return INDArray(t[cond.apply(t)])

    @staticmethod
    def firstIndex(arr, cond, *dims):
        from .ndarray import INDArray
        m = cond.apply(BooleanIndexing._t(arr))
        if not dims:
            nz = m.reshape(-1).nonzero()
            return INDArray(torch.tensor(int(nz[0]) if nz.numel() else -1))
        d = dims[0]
        idx = torch.arange(m.shape[d], device=m.device).reshape([-1 if i == d % m.dim() else 1 for i in range(m.dim())])
        first = torch.where(m, idx, torch.full_like(idx, m.shape[d])).amin(d)
        return INDArray(torch.where(first == m.shape[d], torch.full_like(first, -1), first))

    @staticmethod
    def lastIndex(arr, cond, *dims):
        from .ndarray import INDArray
        m = cond.apply(BooleanIndexing._t(arr))
        if not dims:
            nz = m.reshape(-1).nonzero()
            return INDArray(torch.tensor(int(nz[-1]) if nz.numel() else -1))
        d = dims[0]
        idx = torch.arange(m.shape[d], device=m.device).reshape([-1 if i == d % m.dim() else 1 for i in range(m.dim())])
        return INDArray(torch.where(m, idx, torch.full_like(idx, -1)).amax(d))
