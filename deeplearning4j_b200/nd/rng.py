"""Counter-based random generator with the reference's stream definition.

``libnd4j/include/graph/RandomGenerator.h``: the generator has no sequential state besides two 64-bit words (root state, node
state); the value at position ``index`` is a pure function of (root, node, index), so any op can draw element ``i`` independently
(``relativeT<T>(index)``), and ``rewindH(steps)`` moves the node state on after an op consumed ``steps`` values.  This module
evaluates the same arithmetic for whole index ranges at once (numpy ``uint64`` / ``uint32`` wrap-around), which lets tests and
importers reproduce the reference's random streams for a given seed pair; the training path keeps using torch generators.
"""
from __future__ import annotations

import time

import numpy as np
import torch

_M64 = (1 << 64) - 1
DEFAULT_NODE_SEED = 1298567341


def _u64(v):
    return np.uint64(int(v) & _M64)


class RandomGenerator:
    def __init__(self, rootSeed=0, nodeSeed=0):
        self.setStates(rootSeed, nodeSeed)

    def setStates(self, rootSeed=0, nodeSeed=0):
        self._root = int(rootSeed) & _M64 if rootSeed else int(time.time() * 1000) & _M64
        self._node = int(nodeSeed) & _M64 if nodeSeed else DEFAULT_NODE_SEED

    def setSeed(self, seed):
        self._node = int(seed) & _M64

    def rootState(self): return self._root if self._root < (1 << 63) else self._root - (1 << 64)
    def nodeState(self): return self._node if self._node < (1 << 63) else self._node - (1 << 64)

    # ------------------------------------------------------------------ raw streams
    def xoroshiro32(self, index):
        """uint32 value(s) at ``index`` (scalar or array of non-negative integers)."""
        with np.errstate(over="ignore"):
            idx = np.asarray(index, dtype=np.uint64) + np.uint64(2)
            s0 = _u64(self._root) | (idx * (_u64(self._node) + np.uint64(24243287)))
            s1 = _u64(self._node) ^ (idx * (s0 + np.uint64(723829)))
            half = ((s1 ^ s0) & np.uint64(0xFFFFFFFF)).astype(np.uint32)
            x = half * np.uint32(0x9E3779BB)
            x = (x << np.uint32(5)) | (x >> np.uint32(27))
            return x * np.uint32(5)

    def xoroshiro64(self, index):
        with np.errstate(over="ignore"):
            idx = np.asarray(index, dtype=np.uint64)
            upper = self.xoroshiro32(idx).astype(np.uint64) << np.uint64(32)
            rot = (idx << np.uint64(32)) | (idx >> np.uint64(32))
            return upper + self.xoroshiro32(rot).astype(np.uint64)

    # ------------------------------------------------------------------ typed values
    def relativeFloat(self, index):
        """float32 in [0, 1): the 23 high bits of the 32-bit value become the mantissa of a number in [1, 2)."""
        bits = (np.uint32(0x3F800000) | (self.xoroshiro32(index) >> np.uint32(9))).astype(np.uint32)
        return bits.view(np.float32) - np.float32(1.0)

    def relativeDouble(self, index):
        bits = (np.uint64(0x3FF) << np.uint64(52)) | (self.xoroshiro64(index) >> np.uint64(12))
        return np.asarray(bits, dtype=np.uint64).view(np.float64) - 1.0

    def relativeUInt32(self, index): return self.xoroshiro32(index)
    def relativeUInt64(self, index): return self.xoroshiro64(index)

    def relativeInt(self, index, lo=None, hi=None):
        if lo is None:
            return (self.xoroshiro32(index) & np.uint32(0x7FFFFFFF)).astype(np.int32)
        t = self.relativeFloat(index)
        return (lo + (t * np.float32(hi - lo)).astype(np.int64)).astype(np.int32)

    def relativeT(self, index, lo=0.0, hi=1.0, dtype=torch.float32):
        """Tensor of values in [lo, hi) at the given positions."""
        if dtype == torch.float64:
            v = lo + self.relativeDouble(index) * (hi - lo)
        else:
            v = np.float32(lo) + self.relativeFloat(index) * np.float32(hi - lo)
        return torch.from_numpy(np.ascontiguousarray(v)).to(dtype)

    # ------------------------------------------------------------------ bulk helpers used by random ops
    def uniform(self, shape, lo=0.0, hi=1.0, dtype=torch.float32):
        n = int(np.prod(shape)) if len(shape) else 1
        out = self.relativeT(np.arange(n, dtype=np.uint64), lo, hi, dtype).reshape(tuple(shape))
        self.rewindH(n)
        return out

    def rewindH(self, steps):
        """Advance the node state after ``steps`` values were consumed."""
        s0 = self._node & 0xFFFFFFFF
        s1 = (self._node >> 32) & 0xFFFFFFFF
        s1 ^= s0

        def rotl(x, k):
            return ((x << k) | (x >> (32 - k))) & 0xFFFFFFFF
        v0 = (rotl(s0, 26) ^ s1 ^ ((s1 << 9) & 0xFFFFFFFF)) & 0xFFFFFFFF
        v1 = rotl(s1, 13)
        self._node = ((v1 << 32) | v0) ^ ((int(steps) ^ 0xDEADBEEF) & _M64)
        self._node &= _M64
