"""Small shared types (``nd4j-common``: ``org.nd4j.common.primitives`` / ``org.nd4j.common.base.Preconditions``)."""
from __future__ import annotations

import threading
from collections import defaultdict


class Pair:
    def __init__(self, first=None, second=None):
        self.first, self.second = first, second

    @staticmethod
    def of(a, b): return Pair(a, b)
    makePair = of
    def getFirst(self): return self.first
    def getSecond(self): return self.second
    getKey, getValue, getLeft, getRight = getFirst, getSecond, getFirst, getSecond
    def setFirst(self, v): self.first = v
    def setSecond(self, v): self.second = v
    def __iter__(self): return iter((self.first, self.second))
    def __eq__(self, o): return isinstance(o, Pair) and (self.first, self.second) == (o.first, o.second)
    def __hash__(self): return hash((self.first, self.second))
    def __repr__(self): return f"Pair({self.first!r}, {self.second!r})"


class Triple:
    def __init__(self, first=None, second=None, third=None):
        self.first, self.second, self.third = first, second, third

    @staticmethod
    def of(a, b, c): return Triple(a, b, c)
    def getFirst(self): return self.first
    def getSecond(self): return self.second
    def getThird(self): return self.third
    getLeft, getMiddle, getRight = getFirst, getSecond, getThird
    def __iter__(self): return iter((self.first, self.second, self.third))
    def __eq__(self, o): return isinstance(o, Triple) and tuple(self) == tuple(o)
    def __hash__(self): return hash(tuple(self))
    def __repr__(self): return f"Triple({self.first!r}, {self.second!r}, {self.third!r})"


class AtomicDouble:
    def __init__(self, v=0.0):
        self._v, self._lock = float(v), threading.Lock()

    def get(self): return self._v
    def set(self, v):
        with self._lock:
            self._v = float(v)
    def addAndGet(self, d):
        with self._lock:
            self._v += d
            return self._v
    def getAndAdd(self, d):
        with self._lock:
            old = self._v
            self._v += d
            return old
    def compareAndSet(self, expect, update):
        with self._lock:
            if self._v == expect:
                self._v = float(update)
                return True
            return False
    doubleValue = get
    def __float__(self): return self._v


class AtomicBoolean:
    def __init__(self, v=False):
        self._v, self._lock = bool(v), threading.Lock()

    def get(self): return self._v
    def set(self, v): self._v = bool(v)
    def compareAndSet(self, expect, update):
        with self._lock:
            if self._v == bool(expect):
                self._v = bool(update)
                return True
            return False


class Counter:
    """Element -> float count with totals and arg-max (``org.nd4j.common.primitives.Counter``)."""

    def __init__(self):
        self._m = defaultdict(float)

    def incrementCount(self, k, inc=1.0): self._m[k] += inc
    def incrementAll(self, keys, inc=1.0):
        for k in (keys.keySet() if isinstance(keys, Counter) else keys):
            self._m[k] += keys.getCount(k) if isinstance(keys, Counter) else inc
    def setCount(self, k, v): self._m[k] = float(v)
    def getCount(self, k): return self._m.get(k, 0.0)
    def getProbability(self, k):
        t = self.totalCount()
        return self._m.get(k, 0.0) / t if t else 0.0
    def removeKey(self, k): return self._m.pop(k, None)
    def containsElement(self, k): return k in self._m
    def keySet(self): return set(self._m)
    def keySetSorted(self): return [k for k, _ in sorted(self._m.items(), key=lambda kv: -kv[1])]
    def entrySet(self): return list(self._m.items())
    def totalCount(self): return float(sum(self._m.values()))
    def size(self): return len(self._m)
    def isEmpty(self): return not self._m
    def argMax(self): return max(self._m, key=self._m.get) if self._m else None
    def normalize(self):
        t = self.totalCount()
        if t:
            for k in self._m:
                self._m[k] /= t
    def keepTopNElements(self, n):
        for k in self.keySetSorted()[n:]:
            del self._m[k]
    def dropElementsBelowThreshold(self, th):
        for k in [k for k, v in self._m.items() if v < th]:
            del self._m[k]
    def clear(self): self._m.clear()


class CounterMap:
    """Two-level counter (``CounterMap<F, S>``)."""

    def __init__(self):
        self._m = defaultdict(Counter)

    def incrementCount(self, a, b, inc=1.0): self._m[a].incrementCount(b, inc)
    def setCount(self, a, b, v): self._m[a].setCount(b, v)
    def getCount(self, a, b): return self._m[a].getCount(b) if a in self._m else 0.0
    def getCounter(self, a): return self._m[a]
    def keySet(self): return set(self._m)
    def totalSize(self): return sum(c.size() for c in self._m.values())
    def size(self): return len(self._m)
    def isEmpty(self): return not self._m
    def argMax(self):
        best, bv = None, None
        for a, c in self._m.items():
            b = c.argMax()
            if b is not None and (bv is None or c.getCount(b) > bv):
                best, bv = Pair(a, b), c.getCount(b)
        return best
    def clear(self): self._m.clear()


class Preconditions:
    """Argument / state checks with ``%s`` message templates (``org.nd4j.common.base.Preconditions``)."""

    @staticmethod
    def _msg(msg, args):
        if msg is None:
            return ""
        try:
            return msg % tuple(args) if args else str(msg)
        except TypeError:
            return str(msg) + " " + " ".join(map(str, args))

    @staticmethod
    def checkArgument(cond, msg=None, *args):
        if not cond:
            raise ValueError(Preconditions._msg(msg, args))

    @staticmethod
    def checkState(cond, msg=None, *args):
        if not cond:
            raise RuntimeError(Preconditions._msg(msg, args))

    @staticmethod
    def checkNotNull(obj, msg=None, *args):
        if obj is None:
            raise TypeError(Preconditions._msg(msg or "argument is null", args))
        return obj

    @staticmethod
    def throwEx(msg, *args):
        raise ValueError(Preconditions._msg(msg, args))
