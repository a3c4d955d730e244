"""Host code of the native library under AddressSanitizer + UndefinedBehaviorSanitizer: the sanitizer build is loaded in a child
process (libasan preloaded) and every entry point that needs no device is driven through its argument checks and table lookups.
A sanitizer report makes the child exit non-zero."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import ctypes, os, sys
sys.path.insert(0, %(root)r)
from deeplearning4j_b200.ops import native
from deeplearning4j_b200.utils.launch import LaunchDims
assert native._LIB_PATH.endswith("_asan.so"), native._LIB_PATH
names = LaunchDims.names()
assert len(names) >= 10
for n in names:
    d = LaunchDims.get(n)
    assert d.grid >= 0 and d.block > 0
os.environ["GRID_SIZE_" + names[0].upper()] = "77"
LaunchDims.reload()
assert LaunchDims.get(names[0]).grid == 77
try:
    LaunchDims.get("no_such_kernel_" + "x" * 300)
    raise SystemExit("expected KeyError")
except KeyError:
    pass
lib = ctypes.CDLL(os.path.abspath(native._LIB_PATH))
assert lib.dl4j_abi_version() == 1
lib.dl4j_threshold_msg_ints.restype = ctypes.c_longlong
lib.dl4j_threshold_msg_ints.argtypes = [ctypes.c_longlong, ctypes.c_int]
for n, c in ((1, 1), (1000, 3), (1 << 28, 148 * 4), ((1 << 31) + 5, 1184)):
    assert lib.dl4j_threshold_msg_ints(n, c) > 0
lib.dl4j_step_vars_bytes.restype = ctypes.c_int
assert lib.dl4j_step_vars_bytes() >= 264
lim = (ctypes.c_int * 8)(1024, 232448, 2147483647, 32, 0, 0, 0, 0)       # threads per block, shared memory, grid x, warp size
lib.dl4j_validate_launch.argtypes = [ctypes.c_char_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
free = b"no_table_entry"
assert lib.dl4j_validate_launch(free, 10, 256, 0, lim) == 0
assert lib.dl4j_validate_launch(free, 10, 4096, 0, lim) & 1
assert lib.dl4j_validate_launch(free, 10, 250, 0, lim) & 1
assert lib.dl4j_validate_launch(free, 10, 256, 1 << 30, lim) & 2
assert lib.dl4j_validate_launch(free, 0, 256, 0, lim) & 4
assert lib.dl4j_validate_launch(names[0].encode(), 10, 256, 0, None) == -1
# argument checks of the allocation-free entry point return before any device call
f = lib.dl4j_layer_norm_bwd_noalloc
vp = ctypes.c_void_p
f.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, vp]
f.restype = ctypes.c_int
assert f(None, None, None, None, None, None, None, None, 4, 64, 1, None) != 0
assert f(16, 16, 16, 16, 16, 16, 16, 16, 4, 63, 1, None) != 0          # C %% 8 != 0
assert f(16, 16, 16, 16, 16, 16, 16, 16, 4, 2048, 1, None) != 0        # C > 1024
assert f(18, 16, 16, 16, 16, 16, 16, 16, 4, 64, 1, None) == -6         # misaligned dy
print("SANITIZER_CHILD_OK")
"""


def _libasan():
    r = subprocess.run(["gcc", "-print-file-name=libasan.so"], capture_output=True, text=True)
    p = r.stdout.strip()
    return p if r.returncode == 0 and os.path.isabs(p) and os.path.exists(p) else None


def test_host_code_runs_clean_under_asan_and_ubsan():
    asan = _libasan()
    if asan is None:
        pytest.skip("no libasan on this machine")
    from deeplearning4j_b200.csrc import build
    build.build(asan=True)
    env = dict(os.environ, DL4J_ASAN="1", LD_PRELOAD=asan, ASAN_OPTIONS="detect_leaks=0:abort_on_error=0:exitcode=23",
               UBSAN_OPTIONS="halt_on_error=1:exitcode=24:print_stacktrace=1")
    env.pop("DL4J_DEBUG_BOUNDS", None)
    r = subprocess.run([sys.executable, "-c", CHILD % {"root": ROOT}], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and "SANITIZER_CHILD_OK" in r.stdout, (r.stdout[-1500:] + r.stderr[-3000:])
    assert "AddressSanitizer" not in r.stderr and "runtime error:" not in r.stderr, r.stderr[-3000:]
