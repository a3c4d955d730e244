"""Native workspace arena (``csrc/arena.cu``): a slab with bump allocation per cycle, spill blocks, and a learned high-water mark.
``NativeArena.tensor`` wraps an address as a torch tensor without copying (``__array_interface__`` for host memory,
``__cuda_array_interface__`` for device memory); tensors are valid until the arena's next ``reset``."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

HOST, PINNED, DEVICE = 0, 1, 2
_LIB = None


def _lib():
    global _LIB
    if _LIB is None:
        import os
        from ..ops import native
        l = ctypes.CDLL(os.path.abspath(native._LIB_PATH))
        vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        l.dl4j_arena_create.argtypes, l.dl4j_arena_create.restype = [i32, i64], vp
        l.dl4j_arena_destroy.argtypes, l.dl4j_arena_destroy.restype = [vp], None
        l.dl4j_arena_alloc.argtypes, l.dl4j_arena_alloc.restype = [vp, i64, i32, i32, ctypes.POINTER(i32)], vp
        l.dl4j_arena_reset.argtypes, l.dl4j_arena_reset.restype = [vp], None
        l.dl4j_arena_resize.argtypes, l.dl4j_arena_resize.restype = [vp, i64], i32
        l.dl4j_arena_stats.argtypes, l.dl4j_arena_stats.restype = [vp, ctypes.POINTER(i64)], None
        l.dl4j_arena_base.argtypes, l.dl4j_arena_base.restype = [vp], vp
        _LIB = l
    return _LIB


_NP = {torch.float32: "<f4", torch.float64: "<f8", torch.float16: "<f2", torch.int32: "<i4", torch.int64: "<i8", torch.int16: "<i2",
       torch.int8: "|i1", torch.uint8: "|u1", torch.bool: "|b1", torch.bfloat16: "<i2"}


class _Blob:
    def __init__(self, ptr, shape, typestr, cuda):
        d = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 3 if not cuda else 2, "strides": None}
        if cuda:
            self.__cuda_array_interface__ = d
        else:
            self.__array_interface__ = d


class NativeArena:
    def __init__(self, kind=HOST, initialBytes=0):
        self.kind = int(kind)
        self.h = _lib().dl4j_arena_create(self.kind, int(initialBytes))
        if not self.h:
            raise MemoryError(f"could not create an arena of {initialBytes} bytes (kind {kind})")

    def alloc(self, nbytes, align=256, allowSpill=True):
        sp = ctypes.c_int(0)
        p = _lib().dl4j_arena_alloc(self.h, int(nbytes), int(align), 1 if allowSpill else 0, ctypes.byref(sp))
        if not p:
            raise MemoryError(f"arena: request of {nbytes} bytes does not fit and spilling is off")
        return int(p), bool(sp.value)

    def tensor(self, shape, dtype=torch.float32, allowSpill=True, zero=False):
        shape = tuple(int(s) for s in shape)
        n = int(np.prod(shape)) if shape else 1
        ptr, _ = self.alloc(max(n, 1) * torch.empty(0, dtype=dtype).element_size(), 256, allowSpill)
        if self.kind == DEVICE:
            t = torch.as_tensor(_Blob(ptr, (max(n, 1),), _NP[dtype], True), device="cuda")
        else:
            t = torch.from_numpy(np.asarray(_Blob(ptr, (max(n, 1),), _NP[dtype], False)))
        if dtype == torch.bfloat16:
            t = t.view(torch.bfloat16)
        t = t[:n].reshape(shape)
        if zero:
            t.zero_()
        return t

    def reset(self): _lib().dl4j_arena_reset(self.h)

    def resize(self, nbytes):
        rc = _lib().dl4j_arena_resize(self.h, int(nbytes))
        if rc != 0:
            raise RuntimeError({-2: "the arena can only be resized between cycles", -3: "out of memory"}.get(rc, f"error {rc}"))

    def stats(self):
        out = (ctypes.c_longlong * 8)()
        _lib().dl4j_arena_stats(self.h, out)
        keys = ("capacity", "offset", "cycleBytes", "maxCycleBytes", "spilledBytes", "generation", "cycles", "spillBlocks")
        return dict(zip(keys, (int(v) for v in out)))

    def close(self):
        if self.h:
            _lib().dl4j_arena_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:       # noqa: BLE001
            pass
