"""Launch table with environment overrides and launch validation against explicit device limits (host code only: no GPU)."""
import os

import pytest

LIB = os.path.join(os.path.dirname(__file__), "..", "deeplearning4j_b200", "csrc", "libdl4j_b200.so")
pytestmark = pytest.mark.skipif(not os.path.exists(LIB), reason="native library not built")


def test_table_defaults_and_environment_overrides(monkeypatch):
    from deeplearning4j_b200.utils.launch import LaunchDims
    LaunchDims.reload()
    names = LaunchDims.names()
    assert "BIAS_ACT_BWD" in names and "GEMM_TCGEN05" in names and "LAYER_NORM_FWD" in names
    d = LaunchDims.get("bias_act_bwd")                       # lookup is case-insensitive
    assert (d.grid, d.block, d.fixedBlock) == (6, 256, True)
    monkeypatch.setenv("GRID_SIZE_BIAS_ACT_BWD", "12")
    monkeypatch.setenv("SHARED_MEM_SIZE_BIAS_ACT_BWD", "4096")
    monkeypatch.setenv("GRID_SIZE_LAYER_NORM_FWD", "not-a-number")     # malformed values are ignored
    assert LaunchDims.get("BIAS_ACT_BWD").grid == 6          # resolved values are cached until reload()
    LaunchDims.reload()
    d = LaunchDims.get("BIAS_ACT_BWD")
    assert (d.grid, d.sharedMem) == (12, 4096)
    assert LaunchDims.get("LAYER_NORM_FWD").grid == 4
    with pytest.raises(KeyError):
        LaunchDims.get("no_such_kernel")
    monkeypatch.delenv("GRID_SIZE_BIAS_ACT_BWD")
    monkeypatch.delenv("SHARED_MEM_SIZE_BIAS_ACT_BWD")
    LaunchDims.reload()
    assert LaunchDims.get("BIAS_ACT_BWD").grid == 6


def test_validator_flags_each_limit(monkeypatch):
    from deeplearning4j_b200.utils.launch import DeviceLimits, DeviceValidator, LaunchDims
    LaunchDims.reload()
    v = DeviceValidator(DeviceLimits(maxThreadsPerBlock=1024, maxSharedMemPerBlock=232448, maxGridX=1 << 20, warpSize=32))
    assert v.check("BIAS_ACT_BWD", 888, 256, 8448) == 0
    assert v.check("BIAS_ACT_BWD", 888, 2048, 8448) & v.BLOCK
    assert v.check("BIAS_ACT_BWD", 888, 250, 8448) & v.BLOCK            # not a multiple of the warp size
    assert v.check("BIAS_ACT_BWD", 888, 256, 300000) == v.SHARED_MEM
    assert v.check("BIAS_ACT_BWD", (1 << 20) + 1, 256, 0) == v.GRID
    assert v.check("BIAS_ACT_BWD", 888, 128, 0) == v.FIXED_BLOCK       # the kernel is compiled for 256 threads
    assert v.check("unlisted_kernel", 10, 128, 0) == 0
    assert v.validateTable() == {}
    small = DeviceValidator(DeviceLimits(maxThreadsPerBlock=512, maxSharedMemPerBlock=49152, maxGridX=65535, warpSize=32))
    bad = small.validateTable()
    assert "GEMM_TCGEN05" in bad and "shared memory" in bad["GEMM_TCGEN05"]
    assert "block size" in bad["FLASH_ATTN_BWD"]
