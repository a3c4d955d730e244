"""Launch table and device validation over the native library.

``LaunchDims.get("bias_act_bwd")`` returns the launch parameters a kernel family runs with: the defaults compiled into the
library, overridden by the environment variables ``GRID_SIZE_<NAME>``, ``BLOCK_SIZE_<NAME>`` and ``SHARED_MEM_SIZE_<NAME>``
(reference: libnd4j ``execution/cuda/LaunchDims.h:14-222``).  For the grid-stride kernels ``grid`` is the number of blocks per SM
that the host entry point aims for, and the override takes effect on the next launch; block shapes are compile-time constants,
so a ``BLOCK_SIZE_*`` override is reported by ``DeviceValidator.check`` rather than applied.

``DeviceValidator`` checks a launch against device limits (reference: ``execution/cuda/DeviceValidator.cu``); the limits come from
the current device or are given explicitly, which is how the CPU tests exercise it.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

_LIB = None


def _lib():
    global _LIB
    if _LIB is None:
        from ..ops import native          # the same file the kernels come from (normal, debug-bounds or sanitizer build)
        lib = ctypes.CDLL(os.path.abspath(native._LIB_PATH))
        lib.dl4j_launch_dims.argtypes = [ctypes.c_char_p, ctypes.c_void_p]
        lib.dl4j_launch_dims.restype = ctypes.c_int
        lib.dl4j_launch_dims_name.argtypes = [ctypes.c_int]
        lib.dl4j_launch_dims_name.restype = ctypes.c_char_p
        lib.dl4j_launch_dims_count.restype = ctypes.c_int
        lib.dl4j_launch_dims_reload.restype = None
        lib.dl4j_validate_launch.argtypes = [ctypes.c_char_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        lib.dl4j_validate_launch.restype = ctypes.c_int
        lib.dl4j_device_limits.argtypes = [ctypes.c_void_p]
        lib.dl4j_device_limits.restype = ctypes.c_int
        _LIB = lib
    return _LIB


@dataclass(frozen=True)
class Dims:
    name: str
    grid: int            # blocks per SM for grid-stride kernels; 0 = data dependent
    block: int
    sharedMem: int
    fixedBlock: bool


class LaunchDims:
    @staticmethod
    def names():
        lib = _lib()
        return [lib.dl4j_launch_dims_name(i).decode() for i in range(lib.dl4j_launch_dims_count())]

    @staticmethod
    def get(name) -> Dims:
        out = (ctypes.c_int * 4)()
        if _lib().dl4j_launch_dims(name.encode(), out) != 0:
            raise KeyError(f"no launch table entry for kernel {name!r}")
        return Dims(name.upper(), out[0], out[1], out[2], bool(out[3]))

    @staticmethod
    def reload():
        """Read the environment again on the next query / launch."""
        _lib().dl4j_launch_dims_reload()

    @staticmethod
    def table():
        return {n: LaunchDims.get(n) for n in LaunchDims.names()}


@dataclass(frozen=True)
class DeviceLimits:
    maxThreadsPerBlock: int = 1024
    maxSharedMemPerBlock: int = 232448
    maxGridX: int = 2147483647
    warpSize: int = 32

    @staticmethod
    def current():
        out = (ctypes.c_int * 4)()
        rc = _lib().dl4j_device_limits(out)
        if rc != 0:
            raise RuntimeError(f"device limits unavailable (CUDA error {rc})")
        return DeviceLimits(out[0], out[1], out[2], out[3])


class DeviceValidator:
    BLOCK, SHARED_MEM, GRID, FIXED_BLOCK = 1, 2, 4, 8

    def __init__(self, limits: DeviceLimits | None = None):
        self.limits = limits if limits is not None else DeviceLimits.current()

    def check(self, name, grid, block, sharedMem) -> int:
        """0 when the launch fits; otherwise the OR of BLOCK / SHARED_MEM / GRID / FIXED_BLOCK."""
        l = self.limits
        lim = (ctypes.c_int * 4)(l.maxThreadsPerBlock, l.maxSharedMemPerBlock, l.maxGridX, l.warpSize)
        return _lib().dl4j_validate_launch(name.encode(), int(grid), int(block), int(sharedMem), lim)

    def describe(self, code) -> list[str]:
        names = {self.BLOCK: "block size", self.SHARED_MEM: "shared memory", self.GRID: "grid size",
                 self.FIXED_BLOCK: "block size differs from the kernel's compile-time shape"}
        return [v for k, v in names.items() if code & k]

    def validateTable(self, sms=148):
        """Check every table entry (after environment overrides); returns {name: [problems]} for the entries that do not fit."""
        bad = {}
        for n, d in LaunchDims.table().items():
            code = self.check(n, max(d.grid, 1) * sms, d.block, d.sharedMem)
            if code:
                bad[n] = self.describe(code)
        return bad
