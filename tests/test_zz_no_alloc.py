"""The allocation-free layer-norm backward (``csrc/dl4j_noalloc.h``) called through its exported C symbol.

Collected last on purpose (file name): it has to pass both on its own and after every other GPU test
has used the device, and it checks two calls in a row so that state left in the fixed scratch array by
the first call cannot leak into the second.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

_SO = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "deeplearning4j_b200", "csrc", "libdl4j_b200.so")
_DT = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


@pytest.fixture(scope="module")
def lib():
    so = ctypes.CDLL(os.path.abspath(_SO))
    vp, f_p, i32, i64 = ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    so.dl4j_layer_norm_bwd_noalloc.argtypes = [vp, vp, f_p, f_p, f_p, vp, f_p, f_p, i64, i32, i32, i32, vp]
    so.dl4j_layer_norm_bwd_noalloc.restype = i32
    so.dl4j_layer_norm_bwd.argtypes = [vp, vp, f_p, f_p, f_p, vp, f_p, f_p, i32, i32, i32, vp]
    so.dl4j_layer_norm_bwd.restype = i32
    so.dl4j_bind_device.argtypes = [i32]
    so.dl4j_bind_device.restype = i32
    assert so.dl4j_bind_device(torch.cuda.current_device()) == 0
    return so


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _case(rows, C, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, C, device="cuda", generator=g).to(dtype)
    dy = torch.randn(rows, C, device="cuda", generator=g).to(dtype)
    gain = torch.rand(C, device="cuda", generator=g) + 0.5
    xf = x.float()
    mean = xf.mean(1)
    rstd = (xf.var(1, unbiased=False) + 1e-5).rsqrt()
    return x, dy, gain, mean.contiguous(), rstd.contiguous()


def _existing(lib, x, dy, gain, mean, rstd):
    rows, C = x.shape
    dx = torch.empty_like(x)
    dg = torch.zeros(C, device="cuda")
    db = torch.zeros(C, device="cuda")
    rc = lib.dl4j_layer_norm_bwd(_p(dy), _p(x), _p(gain), _p(mean), _p(rstd), _p(dx), _p(dg), _p(db), rows, C, _DT[x.dtype],
                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    return dx, dg, db


def _noalloc(lib, x, dy, gain, mean, rstd, dg=None, db=None, accumulate=0):
    rows, C = x.shape
    dx = torch.empty_like(x)
    # poison the outputs: the routine must overwrite them without reading when accumulate == 0
    dg = torch.full((C,), float("nan"), device="cuda") if dg is None else dg
    db = torch.full((C,), float("nan"), device="cuda") if db is None else db
    rc = lib.dl4j_layer_norm_bwd_noalloc(_p(dy), _p(x), _p(gain), _p(mean), _p(rstd), _p(dx), _p(dg), _p(db), rows, C,
                                         _DT[x.dtype], accumulate, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    return dx, dg, db


def _torch_ref(x, dy, gain, mean, rstd):
    xh = (x.float() - mean[:, None]) * rstd[:, None]
    d = dy.float()
    dgn = d * gain
    dx = rstd[:, None] * (dgn - dgn.mean(1, keepdim=True) - xh * (dgn * xh).mean(1, keepdim=True))
    return dx, (d * xh).sum(0), d.sum(0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_two_calls_in_a_row_match_existing_entry_point(lib, dtype):
    # the first call fills every scratch slot (296 blocks, widest C); the second uses fewer blocks and a
    # narrower C, so stale partials from call one would show up in its sums if they were read
    for seed, (rows, C) in enumerate([(4096, 1024), (40, 768)]):
        x, dy, gain, mean, rstd = _case(rows, C, dtype, 100 + seed)
        dx0, dg0, db0 = _existing(lib, x, dy, gain, mean, rstd)
        dx1, dg1, db1 = _noalloc(lib, x, dy, gain, mean, rstd)
        torch.cuda.synchronize()
        rdx, rdg, rdb = _torch_ref(x, dy, gain, mean, rstd)
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        torch.testing.assert_close(dx1.float(), dx0.float(), atol=tol, rtol=tol)   # same math as the existing kernel
        torch.testing.assert_close(dx1.float(), rdx, atol=tol * 4, rtol=tol)
        for got, old, ref in ((dg1, dg0, rdg), (db1, db0, rdb)):
            scale = float(ref.abs().max())
            assert float((got - old).abs().max()) <= 1e-4 * scale
            assert float((got - ref).abs().max()) <= 1e-3 * scale


def test_reproducible_and_accumulate(lib):
    x, dy, gain, mean, rstd = _case(3000, 512, torch.bfloat16, 7)
    _, dg_a, db_a = _noalloc(lib, x, dy, gain, mean, rstd)
    _, dg_b, db_b = _noalloc(lib, x, dy, gain, mean, rstd)
    torch.cuda.synchronize()
    assert torch.equal(dg_a, dg_b) and torch.equal(db_a, db_b)       # fixed summation order
    base_g, base_b = torch.ones(512, device="cuda"), torch.full((512,), 2.0, device="cuda")
    _, dg_c, db_c = _noalloc(lib, x, dy, gain, mean, rstd, base_g.clone(), base_b.clone(), accumulate=1)
    torch.cuda.synchronize()
    torch.testing.assert_close(dg_c, dg_a + 1.0)
    torch.testing.assert_close(db_c, db_a + 2.0)


def test_does_not_allocate(lib):
    x, dy, gain, mean, rstd = _case(512, 256, torch.float32, 3)
    _noalloc(lib, x, dy, gain, mean, rstd)                           # first call on this device: set-up done
    dx = torch.empty_like(x)
    dg, db = torch.empty(256, device="cuda"), torch.empty(256, device="cuda")
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        rc = lib.dl4j_layer_norm_bwd_noalloc(_p(dy), _p(x), _p(gain), _p(mean), _p(rstd), _p(dx), _p(dg), _p(db), 512, 256, 2,
                                             0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0


def test_sizes_beyond_the_scratch_are_rejected(lib, capfd):
    x, dy, gain, mean, rstd = _case(8, 2048, torch.float32, 1)
    dx = torch.empty_like(x)
    args = (_p(dy), _p(x), _p(gain), _p(mean), _p(rstd), _p(dx), None, None)
    s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.dl4j_layer_norm_bwd_noalloc(*args, 8, 2048, 2, 0, s) == -6      # wider than the scratch rows
    assert "exceeds" in capfd.readouterr().err
    assert lib.dl4j_layer_norm_bwd_noalloc(*args, 8, 100, 2, 0, s) == -6       # not a multiple of 8
    assert lib.dl4j_layer_norm_bwd_noalloc(*args, 0, 1024, 2, 0, s) == -6      # no rows
    assert lib.dl4j_layer_norm_bwd_noalloc(*args, 8, 1024, 9, 0, s) == -6      # unknown dtype
    # a base pointer that is not 16-byte aligned would make the kernel's vector accesses fault: refused up front
    off = ctypes.c_void_p(x.data_ptr() + 4)
    capfd.readouterr()
    assert lib.dl4j_layer_norm_bwd_noalloc(_p(dy), off, _p(gain), _p(mean), _p(rstd), _p(dx), None, None, 4, 1024, 2, 0, s) == -6
    assert "16-byte aligned" in capfd.readouterr().err
    assert lib.dl4j_layer_norm_bwd_noalloc(_p(dy), _p(x), _p(gain), _p(mean), _p(rstd), off, None, None, 4, 1024, 2, 0, s) == -6
    torch.cuda.synchronize()
