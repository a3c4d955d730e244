"""Scaled dot-product attention on the native kernels.

Reference formulation: ``libnd4j/include/helpers/impl/AttentionHelper.cpp:189-470`` (matmul,
scale, mask add, softmax over the full score matrix, matmul) and the ``dot_product_attention``
/ ``multi_head_dot_product_attention`` ops.  Here every matmul is one launch of the batched
tcgen05 GEMM over strided views of the packed projection buffer (no transposes, no per-head
copies), the scale is folded into the GEMM epilogue, masking + softmax is one in-place fused
kernel, and the backward pass is four batched GEMMs plus one fused softmax-gradient kernel.
The output is produced directly in ``[B, Tq, H, D]`` memory order so the following
``[B*Tq, H*D]`` reshape for the output projection is free.
"""
from __future__ import annotations

import ctypes

import torch

from . import native

_LONG2 = ctypes.c_long * 2


def _ok_view(t):
    """[B, H, T, D] view usable by a rank-4 tensor map: unit inner stride, 16-byte aligned strides."""
    return (t.dim() == 4 and t.stride(3) == 1 and t.stride(2) % 8 == 0 and t.stride(1) % 8 == 0 and t.stride(0) % 8 == 0
            and t.data_ptr() % 16 == 0 and t.shape[3] % 8 == 0)


def _prep(t):
    return t if _ok_view(t) else t.contiguous()


def _bgemm(l, A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, alpha, H, Bn, a_bs, b_bs, c_bs, dtype, out_fp32=0):
    if not hasattr(l.dl4j_gemm_batched, "_typed"):
        vp, i32, lng, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float
        l.dl4j_gemm_batched.argtypes = [vp, vp, vp, i32, i32, i32, lng, lng, lng, i32, i32, i32, i32, f32, i32, i32, i32, i32,
                                        ctypes.POINTER(ctypes.c_long), ctypes.POINTER(ctypes.c_long),
                                        ctypes.POINTER(ctypes.c_long), vp]
        l.dl4j_gemm_batched.restype = ctypes.c_int
        l.dl4j_gemm_batched._typed = True
    bn = 256 if N > 128 else 128
    rc = l.dl4j_gemm_batched(ctypes.c_void_p(A), ctypes.c_void_p(B), ctypes.c_void_p(C), M, N, K, lda, ldb, ldc, a_mn, b_mn,
                             native._DT[dtype], out_fp32, float(alpha), bn, native.num_sms(), H, Bn, _LONG2(*a_bs),
                             _LONG2(*b_bs), _LONG2(*c_bs), native._stream())
    native._check(rc, "dl4j_gemm_batched")


def _typed_softmax(l):
    if not hasattr(l.dl4j_attn_softmax_fwd, "_typed"):
        vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        l.dl4j_attn_softmax_fwd.argtypes = [vp, vp, i64, i32, i32, i32, vp]
        l.dl4j_attn_softmax_fwd.restype = ctypes.c_int
        l.dl4j_attn_softmax_bwd.argtypes = [vp, vp, i64, i32, f32, i32, vp]
        l.dl4j_attn_softmax_bwd.restype = ctypes.c_int
        l.dl4j_attn_softmax_fwd._typed = True


class _AttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, key_mask, scale, dropout_p=0.0):
        l = native.require()
        _typed_softmax(l)
        q, k, v = _prep(q), _prep(k), _prep(v)
        Bn, H, Tq, D = q.shape
        Tk = k.shape[2]
        dt = q.dtype
        ctx.flash = (USE_FLASH or dropout_p > 0.0) and flash_supported(q, k, v)
        if ctx.flash:
            # fused kernel: the score matrix stays in tensor memory; only O and the row log-sum-exp are written
            seed = _next_dropout_seed(q.device) if dropout_p > 0.0 else None
            O, lse = flash_forward(q, k, v, key_mask, scale, dropout_p, seed)
            mk = key_mask.to(torch.float32).contiguous() if key_mask is not None else None
            ctx.save_for_backward(q, k, v, O, lse, mk, seed)
            ctx.scale, ctx.dropout_p = scale, float(dropout_p)
            return O.permute(0, 2, 1, 3)
        if dropout_p > 0.0:
            raise RuntimeError("attention dropout needs the fused kernels (head size 64, key length a multiple of 128)")
        P = torch.empty((Bn, H, Tq, Tk), dtype=dt, device=q.device)
        # S = scale * Q K^T
        _bgemm(l, q.data_ptr(), k.data_ptr(), P.data_ptr(), Tq, Tk, D, q.stride(2), k.stride(2), Tk, 0, 0, scale, H, Bn,
               (q.stride(1), q.stride(0)), (k.stride(1), k.stride(0)), (Tq * Tk, H * Tq * Tk), dt)
        mk = None
        if key_mask is not None:
            mk = key_mask.to(torch.float32).contiguous()
        rc = l.dl4j_attn_softmax_fwd(native._ptr(P), native._ptr(mk), Bn * H * Tq, Tk, H * Tq, native._DT[dt], native._stream())
        native._check(rc, "dl4j_attn_softmax_fwd")
        # O = P V, written as [B, Tq, H, D]
        O = torch.empty((Bn, Tq, H, D), dtype=dt, device=q.device)
        _bgemm(l, P.data_ptr(), v.data_ptr(), O.data_ptr(), Tq, D, Tk, Tk, v.stride(2), H * D, 0, 1, 1.0, H, Bn,
               (Tq * Tk, H * Tq * Tk), (v.stride(1), v.stride(0)), (D, Tq * H * D), dt)
        ctx.save_for_backward(q, k, v, P)
        ctx.scale = scale
        return O.permute(0, 2, 1, 3)

    @staticmethod
    def backward(ctx, dO):
        l = native.require()
        if ctx.flash:
            return _flash_backward(ctx, dO)
        q, k, v, P = ctx.saved_tensors
        Bn, H, Tq, D = q.shape
        Tk = k.shape[2]
        dt = q.dtype
        dO = _prep(dO)
        same_len = Tq == Tk
        # packed gradient buffer [B, T, 3, H, D] when possible so the three results share one allocation
        if same_len:
            dqkv = torch.empty((Bn, Tq, 3, H, D), dtype=dt, device=q.device)
            dq_t, dk_t, dv_t = dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2]          # [B, T, H, D] views
        else:
            dq_t = torch.empty((Bn, Tq, H, D), dtype=dt, device=q.device)
            dk_t = torch.empty((Bn, Tk, H, D), dtype=dt, device=q.device)
            dv_t = torch.empty((Bn, Tk, H, D), dtype=dt, device=q.device)
        pbs = (Tq * Tk, H * Tq * Tk)

        def obs(t):   # batch strides (head, example) and row stride of a [B, T, H, D] output view
            return (t.stride(2), t.stride(0)), t.stride(1)
        # dV = P^T dO
        cbs, ldc = obs(dv_t)
        _bgemm(l, P.data_ptr(), dO.data_ptr(), dv_t.data_ptr(), Tk, D, Tq, Tk, dO.stride(2), ldc, 1, 1, 1.0, H, Bn,
               pbs, (dO.stride(1), dO.stride(0)), cbs, dt)
        # dP = dO V^T
        dP = torch.empty_like(P)
        _bgemm(l, dO.data_ptr(), v.data_ptr(), dP.data_ptr(), Tq, Tk, D, dO.stride(2), v.stride(2), Tk, 0, 0, 1.0, H, Bn,
               (dO.stride(1), dO.stride(0)), (v.stride(1), v.stride(0)), pbs, dt)
        rc = l.dl4j_attn_softmax_bwd(native._ptr(P), native._ptr(dP), Bn * H * Tq, Tk, float(ctx.scale), native._DT[dt],
                                     native._stream())
        native._check(rc, "dl4j_attn_softmax_bwd")
        # dQ = dS K
        cbs, ldc = obs(dq_t)
        _bgemm(l, dP.data_ptr(), k.data_ptr(), dq_t.data_ptr(), Tq, D, Tk, Tk, k.stride(2), ldc, 0, 1, 1.0, H, Bn,
               pbs, (k.stride(1), k.stride(0)), cbs, dt)
        # dK = dS^T Q
        cbs, ldc = obs(dk_t)
        _bgemm(l, dP.data_ptr(), q.data_ptr(), dk_t.data_ptr(), Tk, D, Tq, Tk, q.stride(2), ldc, 1, 1, 1.0, H, Bn,
               pbs, (q.stride(1), q.stride(0)), cbs, dt)
        return dq_t.permute(0, 2, 1, 3), dk_t.permute(0, 2, 1, 3), dv_t.permute(0, 2, 1, 3), None, None, None


def attention(q, k, v, mask, scale, dropout_p=0.0):
    """q, k, v: [B, H, T, D]; ``mask``: None or a [B, Tk] key mask (non-zero = attend); ``dropout_p``: probability of dropping an
    attention weight (training).  Returns None when the case is not covered by the native kernels.

    Head sizes below 64 run on the fused head-size-64 kernels with zero-padded heads (Q K^T is unchanged by zero columns, the
    padded columns of V give output columns that are sliced away), so no score matrix is materialised for them either."""
    if not native.available() or q.dim() != 4 or q.dtype not in (torch.bfloat16, torch.float16):
        return None
    if mask is not None and (mask.dim() != 2 or mask.shape[0] != q.shape[0] or mask.shape[1] != k.shape[2]):
        return None
    D, Tk, Tq = q.shape[3], k.shape[2], q.shape[2]
    scale = float(scale) if scale is not None else D ** -0.5
    if D < 64 and D % 8 == 0 and q.dtype == torch.bfloat16 and Tk % 128 == 0 and Tk == v.shape[2] and q.shape[:2] == k.shape[:2]:
        pad = (0, 64 - D)
        qp, kp, vp = (torch.nn.functional.pad(t, pad) for t in (q, k, v))
        return _AttentionFn.apply(qp, kp, vp, mask, scale, float(dropout_p))[..., :D]
    fused = flash_supported(q, k, v)
    if dropout_p > 0.0 and not fused:
        return None
    if D % 8 or Tk % 8 or Tq % 8 or (Tk > 1024 and not fused):
        return None
    return _AttentionFn.apply(q, k, v, mask, scale, float(dropout_p))


# Dropout seeds live on the device: every fused forward call with dropout takes a private copy of the running seed and
# advances it, both with device-side operations, so a captured CUDA graph draws a new mask at every replay; the backward pass
# reads the forward's copy.
_DROPOUT_SEED = {}


def set_dropout_seed(seed, device=None):
    """(Re)starts the attention-dropout seed sequence of ``device`` (default: the current CUDA device)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    _DROPOUT_SEED[device] = torch.tensor([int(seed) & 0x7fffffffffffffff], dtype=torch.int64, device=device)


def _next_dropout_seed(device):
    state = _DROPOUT_SEED.get(device)
    if state is None:
        set_dropout_seed(torch.initial_seed(), device)
        state = _DROPOUT_SEED[device]
    mine = state.clone()
    state.add_(0x9E3779B97F4A7C15 & 0x3fffffffffffffff)      # any odd stride: consecutive calls never share a Philox key
    return mine


_LONG3 = ctypes.c_long * 3
_DQ_ACC = {}
USE_FLASH = True      # False: batched GEMMs + separate softmax kernels with a materialised score matrix (cross-check path)


def _flash_backward(ctx, dO):
    l = native.require()
    if not hasattr(l.dl4j_flash_attn_bwd, "_typed"):
        vp, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        lp = ctypes.POINTER(ctypes.c_long)
        l.dl4j_flash_attn_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, lp, lp, lp, lp, ctypes.c_long, ctypes.c_long, f32,
                                          f32, vp, vp]
        l.dl4j_flash_attn_bwd.restype = ctypes.c_int
        l.dl4j_attn_dvec.argtypes = [vp, lp, vp, vp, i32, i32, i32, vp]
        l.dl4j_attn_dvec.restype = ctypes.c_int
        l.dl4j_attn_dq_finish.argtypes = [vp, vp, ctypes.c_long, ctypes.c_long, i32, i32, i32, vp]
        l.dl4j_attn_dq_finish.restype = ctypes.c_int
        l.dl4j_flash_attn_bwd._typed = True
    q, k, v, O, lse, mk, seed = ctx.saved_tensors
    Bn, H, Tq, D = q.shape
    Tk = k.shape[2]
    dO = _prep(dO)                                           # [B, H, Tq, D] view
    def st(t):
        return _LONG3(t.stride(0), t.stride(1), t.stride(2))
    # D_r = sum_d dO * O per query row, laid out like the log-sum-exp
    dvec = torch.empty((Bn, H, Tq), dtype=torch.float32, device=q.device)
    rc = l.dl4j_attn_dvec(native._ptr(dO), st(dO), native._ptr(O), native._ptr(dvec), Bn, H, Tq, native._stream())
    native._check(rc, "dl4j_attn_dvec")
    # fp32 dQ accumulator: allocated zeroed once per shape, the finishing kernel clears it again after reading it
    key = (q.device, Bn, H, Tq)
    dq_acc = _DQ_ACC.get(key)
    if dq_acc is None:
        dq_acc = _DQ_ACC[key] = torch.zeros((Bn, H, Tq, D), dtype=torch.float32, device=q.device)
    same_len = Tq == Tk
    if same_len:
        # one packed [B, T, 3, H, D] gradient buffer, so the gradient of the fused q/k/v projection is a plain view
        dqkv = torch.empty((Bn, Tq, 3, H, D), dtype=q.dtype, device=q.device)
        dq_t, dk_t, dv_t = dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2]
    else:
        dq_t = torch.empty((Bn, Tq, H, D), dtype=q.dtype, device=q.device)
        dk_t = torch.empty((Bn, Tk, H, D), dtype=q.dtype, device=q.device)
        dv_t = torch.empty((Bn, Tk, H, D), dtype=q.dtype, device=q.device)

    rc = l.dl4j_flash_attn_bwd(native._ptr(q), native._ptr(k), native._ptr(v), native._ptr(dO), native._ptr(lse), native._ptr(dvec),
                               native._ptr(mk), native._ptr(dq_acc), native._ptr(dk_t), native._ptr(dv_t), Bn, H, Tq, Tk,
                               st(q), st(k), st(v), st(dO), dk_t.stride(0), dk_t.stride(1), float(ctx.scale), float(ctx.dropout_p),
                               native._ptr(seed), native._stream())
    native._check(rc, "dl4j_flash_attn_bwd")
    rc = l.dl4j_attn_dq_finish(native._ptr(dq_acc), native._ptr(dq_t), dq_t.stride(0), dq_t.stride(1), Bn, H, Tq, native._stream())
    native._check(rc, "dl4j_attn_dq_finish")
    return dq_t.permute(0, 2, 1, 3), dk_t.permute(0, 2, 1, 3), dv_t.permute(0, 2, 1, 3), None, None, None


def flash_supported(q, k, v):
    return (native.available() and q.dtype == torch.bfloat16 and q.dim() == 4 and q.shape[3] == 64 and k.shape[2] >= 128
            and k.shape[2] % 128 == 0 and k.shape[2] == v.shape[2] and q.shape[:2] == k.shape[:2] and v.shape[3] == 64)


def flash_forward(q, k, v, key_mask, scale, dropout_p=0.0, seed=None):
    """Fused attention forward: returns (out [B, Tq, H, 64] bf16, lse [B, H, Tq] fp32).  q, k, v: [B, H, T, 64] views."""
    l = native.require()
    if not hasattr(l.dl4j_flash_attn_fwd, "_typed"):
        vp, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        lp = ctypes.POINTER(ctypes.c_long)
        l.dl4j_flash_attn_fwd.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, lp, lp, lp, f32, f32, vp, vp]
        l.dl4j_flash_attn_fwd.restype = ctypes.c_int
        l.dl4j_flash_attn_fwd._typed = True
    q, k, v = _prep(q), _prep(k), _prep(v)
    Bn, H, Tq, D = q.shape
    Tk = k.shape[2]
    out = torch.empty((Bn, Tq, H, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((Bn, H, Tq), dtype=torch.float32, device=q.device)
    mk = key_mask.to(torch.float32).contiguous() if key_mask is not None else None

    def st(t):
        return _LONG3(t.stride(0), t.stride(1), t.stride(2))
    rc = l.dl4j_flash_attn_fwd(native._ptr(q), native._ptr(k), native._ptr(v), native._ptr(out), native._ptr(lse), native._ptr(mk),
                               Bn, H, Tq, Tk, st(q), st(k), st(v), float(scale), float(dropout_p), native._ptr(seed), native._stream())
    native._check(rc, "dl4j_flash_attn_fwd")
    return out, lse
