"""ctypes bindings to the in-tree sm_100a library (``csrc/libdl4j_b200.so``) and the autograd
functions that put its kernels on the training path.

The library exports a plain C ABI over raw device pointers + a CUDA stream, so loading it does
not depend on torch's C++ ABI and building it takes seconds.  On a machine with a GPU the
library is mandatory: ``require()`` raises if it cannot be loaded, so a silent torch fallback
cannot masquerade as the native path.
"""
from __future__ import annotations

import ctypes
import os
import struct
import threading

import numpy as np
import torch

_LIB = None
_LIB_ERR = None
_LOCK = threading.Lock()
# DL4J_DEBUG_BOUNDS=1 loads the build whose kernels check their element offsets (``csrc/build.py --debug-bounds``), DL4J_ASAN=1 the
# build whose host code runs under AddressSanitizer / UBSan (``--asan``; the process needs libasan preloaded).
_LIB_FLAVOUR = "dbg" if os.environ.get("DL4J_DEBUG_BOUNDS", "0") == "1" else "asan" if os.environ.get("DL4J_ASAN", "0") == "1" else ""
_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc",
                         "libdl4j_b200" + ("_" + _LIB_FLAVOUR if _LIB_FLAVOUR else "") + ".so")

LAUNCHES = 0     # number of native kernel launches issued by this process (bench.py reports it)

_ACT_IDS = {"ActivationIdentity": 0, "ActivationReLU": 1, "ActivationGELU": 6, "ActivationSigmoid": 4, "ActivationTanH": 5}


def _load():
    global _LIB, _LIB_ERR
    with _LOCK:
        if _LIB is not None or _LIB_ERR is not None:
            return _LIB
        path = os.path.abspath(_LIB_PATH)
        if not os.path.exists(path):
            _LIB_ERR = f"{path} not built (run python -m deeplearning4j_b200.csrc.build)"
            return None
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            _LIB_ERR = str(e)
            return None
        vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        lng = ctypes.c_long
        sig = {
            "dl4j_gemm": [vp, vp, vp, vp, vp, vp, i32, i32, i32, lng, lng, lng, lng, lng, i32, i32, i32, i32, i32, i32,
                          i32, i32, f32, i32, i32, vp],
            "dl4j_fused_update": [vp, vp, vp, vp, vp, vp, i32, vp, vp, i32, f32, i32, vp],
            "dl4j_cast_f32_bf16": [vp, vp, i64, vp],
            "dl4j_threshold_encode": [vp, i64, f32, vp, i32, vp],
            "dl4j_threshold_decode": [vp, i32, vp, i64, f32, i32, vp],
            "dl4j_bitmap_encode": [vp, i64, f32, vp, vp],
            "dl4j_bitmap_decode": [vp, vp, i64, f32, vp],
            "dl4j_layer_norm_fwd": [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, f32, i32, vp],
            "dl4j_layer_norm_bwd": [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp],
            "dl4j_softmax_xent": [vp, vp, vp, vp, vp, i32, i32, i64, i32, i32, vp],
            "dl4j_scatter_add_rows": [vp, vp, vp, i64, i32, i64, i64, i32, vp],
            "dl4j_softmax_xent_fwd": [vp, vp, vp, vp, vp, vp, i32, i32, i64, i32, i32, vp],
            "dl4j_softmax_xent_bwd": [vp, vp, vp, vp, vp, vp, vp, i32, i32, i64, i64, i32, i32, vp],
            "dl4j_lstm_cell_fwd": [vp, vp, vp, vp, vp, i32, i32, i32, vp],
            "dl4j_lstm_cell_bwd": [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp],
            "dl4j_lstm_seq_fwd": [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, vp],
            "dl4j_lstm_seq_bwd": [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, vp],
            "dl4j_transpose16": [vp, vp, i32, i32, vp],
            "dl4j_bias_act_bwd": [vp, vp, vp, vp, i32, i32, i32, i32, vp],
            "dl4j_bn_fwd_train": [vp, vp, vp, vp, vp, vp, i32, f32, f32, i32, vp, vp, vp, vp, vp, i64, i32, vp],
            "dl4j_bn_apply": [vp, vp, vp, vp, i32, vp, i64, i32, vp],
            "dl4j_bn_bwd": [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, vp],
            "dl4j_add_relu": [vp, vp, vp, i64, vp],
            "dl4j_maxpool_fwd": [vp, vp, vp, vp, vp],
            "dl4j_maxpool_bwd": [vp, vp, vp, vp, vp],
            "dl4j_subsample": [vp, vp, vp, i32, vp],
            "dl4j_conv_weight_to_cl": [vp, vp, i32, i32, i32, vp],
            "dl4j_conv_wgrad_from_cl": [vp, vp, i32, i32, i32, vp],
            "dl4j_read_status": [i32],
            "dl4j_num_sms": [],
            "dl4j_bind_device": [i32],
            "dl4j_abi_version": [],
        }
        for name, args in sig.items():
            fn = getattr(lib, name, None)
            if fn is not None:
                fn.argtypes = args
                fn.restype = ctypes.c_int
        for name in dir(lib):
            pass
        _LIB = lib
        return lib


def lib():
    return _load()


def available() -> bool:
    return torch.cuda.is_available() and _load() is not None


def require():
    """Fail loudly when a GPU is present but the native library is not."""
    if torch.cuda.is_available() and _load() is None:
        raise RuntimeError(f"deeplearning4j_b200 native library unavailable on a GPU machine: {_LIB_ERR}")
    return _LIB


def load_error():
    _load()
    return _LIB_ERR


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    """Current torch stream handle; also binds the current device's context to this thread for the
    library's own CUDA runtime instance (autograd worker threads may not have one bound yet)."""
    rc = _LIB.dl4j_bind_device(torch.cuda.current_device())
    if rc != 0:
        raise RuntimeError(f"dl4j_bind_device failed with CUDA error {rc}")
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(rc, what):
    global LAUNCHES
    LAUNCHES += 1
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


def check_status(reset=True):
    """Raise if any bounded device-side wait expired since the last check (synchronises)."""
    l = require()
    if l is None:
        return 0
    v = l.dl4j_read_status(1 if reset else 0)
    if _LIB_FLAVOUR == "dbg":
        rec = debug_bounds(reset)
        if rec["failures"]:
            raise RuntimeError(f"debug bounds check failed {rec['failures']} time(s); first: source line {rec['line']}, "
                               f"offset {rec['offset']}, extent {rec['extent']}")
    if v != 0:
        names = {1: "TMA producer wait", 2: "MMA wait", 3: "epilogue wait", 4: "peer wait", 5: "index out of bounds"}
        raise RuntimeError(f"device-side bounded wait/ check failed: {names.get(v, v)}")
    return v


def debug_bounds(reset=True):
    """The debug-bounds build's record: number of out-of-range offsets the kernels skipped since the last reset, and the source
    line, offset and extent of the first (synchronises).  ``None`` in the normal build."""
    l = require()
    if l is None:
        return None
    out = (ctypes.c_ulonglong * 4)()
    l.dl4j_debug_bounds.argtypes = [ctypes.c_void_p, ctypes.c_int]
    l.dl4j_debug_bounds.restype = ctypes.c_int
    if l.dl4j_debug_bounds(out, 1 if reset else 0) != 0:
        return None
    off = out[2] - (1 << 64) if out[2] >= (1 << 63) else out[2]
    return {"failures": int(out[0]), "line": int(out[1]), "offset": int(off), "extent": int(out[3])}


_DT = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}
_NUM_SMS = None


def num_sms():
    global _NUM_SMS
    if _NUM_SMS is None:
        _NUM_SMS = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _NUM_SMS


# =========================================================================== GEMM
def _operand_a(a):
    """logical [M, K] -> (tensor, mn_major flag, leading dim) or None."""
    if a.stride(1) == 1 and a.stride(0) % 8 == 0 and a.stride(0) >= a.shape[1] and a.data_ptr() % 16 == 0:
        return a, 0, a.stride(0)
    if a.stride(0) == 1 and a.stride(1) % 8 == 0 and a.stride(1) >= a.shape[0] and a.data_ptr() % 16 == 0:
        return a, 1, a.stride(1)
    return None


def _operand_b(b):
    """logical [K, N] -> (tensor, mn_major flag, leading dim) or None."""
    if b.stride(0) == 1 and b.stride(1) % 8 == 0 and b.stride(1) >= b.shape[0] and b.data_ptr() % 16 == 0:
        return b, 0, b.stride(1)       # stored [N, K]
    if b.stride(1) == 1 and b.stride(0) % 8 == 0 and b.stride(0) >= b.shape[1] and b.data_ptr() % 16 == 0:
        return b, 1, b.stride(0)       # stored [K, N]
    return None


def gemm_supported(a, b) -> bool:
    if not available() or a.dim() != 2 or b.dim() != 2 or a.dtype != b.dtype or a.dtype not in (torch.bfloat16, torch.float16):
        return False
    if a.shape[1] != b.shape[0] or min(a.shape[0], a.shape[1], b.shape[1]) == 0:
        return False
    return _operand_a(a) is not None and _operand_b(b) is not None


def _pick_block_n(M, N, splits=1):
    sms = num_sms()
    best, best_cost = 256, None
    for bn in (256, 128):
        tiles = ((M + 127) // 128) * ((N + bn - 1) // bn) * splits
        waves = (tiles + sms - 1) // sms
        cost = waves * bn * (1.0 if bn == 256 else 1.08)     # 128-wide tiles pay a little more per column
        if best_cost is None or cost < best_cost:
            best, best_cost = bn, cost
    return best


_PAIR_MODE = os.environ.get("DL4J_GEMM_PAIR", "0")     # 0 | 1: 256x256 tiles on CTA pairs (cta_group::2) for large problems


def _use_pair(M, N, K, splits):
    """Whether a GEMM runs on CTA pairs (``csrc/gemm_pair_tcgen05.cu``).  Off unless requested: measured on the BERT-base shapes
    the pair kernel ties the single-CTA kernel (30 / 75 / 71 / 58 us against 30 / 71 / 71 / 54 us for out / ffn1 / ffn2 / qkv) and
    loses on 8192^3 (1058 against 790 us): the kernels are bound by the depth of the shared-memory ring over the load latency,
    not by the shared-memory bandwidth a pair saves, and the pair's "stage landed" hand-off between the CTAs adds to that latency."""
    if _PAIR_MODE != "1":
        return False
    return M >= 2048 and N >= 512 and ((M + 255) // 256) * ((N + 255) // 256) * max(splits, 1) >= 74


def gemm_raw(a, b, out=None, bias=None, act=0, aux=None, residual=None, out_dtype=None, atomic=False, splits=1,
             alpha=1.0, block_n=None, pair=None, res_act=0):
    """out[M,N] = act(alpha * a @ b + bias) + residual with a logical [M,K], b logical [K,N].  With ``res_act`` (an activation id)
    ``residual`` holds pre-activations z and the result is multiplied by act'(z) instead: a data-gradient GEMM that writes dz."""
    l = require()
    if res_act:
        if residual is None or act:
            raise ValueError("res_act needs the pre-activations as `residual` and no forward activation")
        act = int(res_act) << 8
        pair = False
    oa, ob = _operand_a(a), _operand_b(b)
    if oa is None or ob is None:
        raise ValueError("operand layout not addressable by TMA (need unit stride in one dim, 16-byte alignment)")
    M, K = a.shape
    N = b.shape[1]
    if out is None:
        out_dtype = out_dtype or a.dtype
        out = (torch.zeros if atomic else torch.empty)((M, N), dtype=out_dtype, device=a.device)
    if out.stride(1) != 1:
        raise ValueError("output must be row-major")
    out_fp32 = 1 if out.dtype == torch.float32 else 0
    if not out_fp32 and out.dtype != a.dtype:
        raise ValueError("output dtype must be the input dtype or float32")
    kb = (K + 63) // 64
    splits = max(1, min(int(splits), kb))
    if splits > 1 and not (atomic and out_fp32):
        splits = 1
    bn = block_n or _pick_block_n(M, N, splits)
    bias_fp32 = 1 if (bias is not None and bias.dtype == torch.float32) else 0
    if bias is not None and not bias_fp32 and bias.dtype != a.dtype:
        bias = bias.to(a.dtype)
    if bias is not None and not bias.is_contiguous():
        bias = bias.contiguous()
    if pair is None:
        pair = block_n is None and _use_pair(M, N, K, splits)
    if pair:
        if not getattr(l, "_pair_typed", False):
            vp, i32, lng, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float
            l.dl4j_gemm_pair.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, lng, lng, lng, lng, lng, i32, i32, i32, i32, i32, i32,
                                         i32, i32, f32, i32, vp]
            l.dl4j_gemm_pair.restype = i32
            l._pair_typed = True
        rc = l.dl4j_gemm_pair(_ptr(oa[0]), _ptr(ob[0]), _ptr(out), _ptr(aux), _ptr(bias), _ptr(residual), M, N, K, oa[2], ob[2],
                              out.stride(0), 0 if aux is None else aux.stride(0), 0 if residual is None else residual.stride(0),
                              oa[1], ob[1], _DT[a.dtype], bias_fp32, out_fp32, int(act), 1 if atomic else 0, splits, float(alpha),
                              num_sms(), _stream())
        _check(rc, "dl4j_gemm_pair")
        return out
    rc = l.dl4j_gemm(_ptr(oa[0]), _ptr(ob[0]), _ptr(out), _ptr(aux), _ptr(bias), _ptr(residual), M, N, K, oa[2], ob[2],
                     out.stride(0), 0 if aux is None else aux.stride(0), 0 if residual is None else residual.stride(0),
                     oa[1], ob[1], _DT[a.dtype], bias_fp32, out_fp32, int(act), 1 if atomic else 0, splits, float(alpha),
                     bn, num_sms(), _stream())
    _check(rc, "dl4j_gemm")
    return out


class _MatmulFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return gemm_raw(a, b)

    @staticmethod
    def backward(ctx, dy):
        a, b = ctx.saved_tensors
        dy = dy if dy.stride(1) == 1 or dy.stride(0) == 1 else dy.contiguous()
        da = db = None
        if ctx.needs_input_grad[0]:
            da = gemm(dy, b.t())
        if ctx.needs_input_grad[1]:
            db = gemm(a.t(), dy)
        return da, db


def gemm(a, b):
    """Differentiable 2-D matmul on the tcgen05 kernel (falls back to torch for odd layouts)."""
    if not gemm_supported(a, b):
        return torch.matmul(a, b)
    if torch.is_grad_enabled() and (a.requires_grad or b.requires_grad):
        return _MatmulFn.apply(a, b)
    return gemm_raw(a, b)


# =========================================================================== Linear (+bias +activation)
def _act_id(activation):
    if activation is None:
        return 0
    name = type(activation).__name__
    if name == "ActivationGELU":
        return 3 if getattr(activation, "precise", False) else 6      # tanh form / x * sigmoid(1.702 x)
    if name == "ActivationReLU":
        if getattr(activation, "max", None) is not None or getattr(activation, "threshold", None) or getattr(activation, "negativeSlope", None):
            return None
        return 1
    return _ACT_IDS.get(name)


def _wgrad_splits(n_out_tiles, K):
    sms = num_sms()
    if n_out_tiles >= sms:
        return 1
    return max(1, min((K + 63) // 64, (2 * sms) // max(n_out_tiles, 1), 32))


def _bias_grad_buffer(b, needed, N, device):
    """(accumulator, returned gradient): the bias' own fp32 ``.grad`` when the kernels may add into it, else a fresh buffer."""
    if b is None or not needed:
        return None, None
    if b.is_leaf and b.grad is not None and b.grad.dtype == torch.float32 and b.grad.is_contiguous():
        return b.grad, None
    acc = torch.zeros(N, dtype=torch.float32, device=device)
    return acc, acc


def _weight_grad(W, x, dz):
    """dW of ``y = x @ W`` accumulated into ``W.grad`` when its layout allows (returns None), else returned in W's layout."""
    M, N = dz.shape
    nIn = x.shape[1]
    tiles = ((N + 127) // 128) * ((nIn + 255) // 256)
    splits = _wgrad_splits(tiles, M)
    g = W.grad if (W.is_leaf and W.grad is not None) else None
    if g is not None and g.dim() == 4 and g.shape[2] == 1 and g.shape[3] == 1 and g.is_contiguous():
        g = g.view(g.shape[0], g.shape[1]).t()      # 1x1 convolution kernel [nOut, nIn, 1, 1]: same memory as an 'f' dense weight
    if g is not None and g.dtype == torch.float32 and g.dim() == 2 and g.stride(0) == 1 and g.stride(1) == nIn \
            and g.data_ptr() % 16 == 0 and nIn % 4 == 0:
        gemm_raw(dz.t(), x, out=g.t(), atomic=True, splits=splits)
        return None
    if g is not None and g.dtype == torch.float32 and g.dim() == 2 and g.is_contiguous() and g.data_ptr() % 16 == 0 and N % 4 == 0:
        # row-major [nIn, nOut] master (SameDiff variables): dW = x^T dz accumulated in place
        tiles2 = ((nIn + 127) // 128) * ((N + 255) // 256)
        gemm_raw(x.t(), dz, out=g, atomic=True, splits=_wgrad_splits(tiles2, M))
        return None
    dWt = gemm_raw(dz.t(), x, out_dtype=torch.float32, atomic=True, splits=splits)
    return dWt.reshape(W.shape).to(W.dtype) if W.dim() == 4 else dWt.t().to(W.dtype)


def _fwd_bias(b, dtype):
    """(bias operand for the forward GEMM, master the gradient goes to)."""
    if b is None:
        return None, None
    b_fwd = b if b.dtype == dtype else getattr(b, "_lp", None)
    if b_fwd is not None:
        b_fwd = b_fwd.detach()
    master = getattr(b, "_master", b)
    if b_fwd is None:
        b_fwd = master
    return b_fwd.reshape(-1), master


class _MlpFn(torch.autograd.Function):
    """y = act(x @ W1 + b1) @ W2 + b2 as one autograd node.  Forward: two GEMMs (the first saves its pre-activation z1 from the
    epilogue).  Backward: the data-gradient GEMM of the second layer multiplies by act'(z1) in its epilogue and writes dz1
    directly, so the separate pass that read dy1 and z1 and wrote dz1 disappears; the bias gradient of the first layer is a
    column sum over dz1 alone."""

    @staticmethod
    def forward(ctx, x, W1, b1, W2, b2, act, W1_lp, W2_lp):
        z1 = torch.empty((x.shape[0], W1_lp.shape[1]), dtype=x.dtype, device=x.device)
        b1_fwd, b1_m = _fwd_bias(b1, x.dtype)
        b2_fwd, b2_m = _fwd_bias(b2, x.dtype)
        y1 = gemm_raw(x, W1_lp, bias=b1_fwd, act=act, aux=z1)
        y2 = gemm_raw(y1, W2_lp, bias=b2_fwd)
        ctx.act = act
        ctx.refs = (getattr(W1, "_master", W1), b1_m, getattr(W2, "_master", W2), b2_m)
        ctx.save_for_backward(x, W1_lp, W2_lp, z1, y1)
        return y2

    @staticmethod
    def backward(ctx, dy2):
        x, W1_lp, W2_lp, z1, y1 = ctx.saved_tensors
        W1, b1, W2, b2 = ctx.refs
        l = require()
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        M, N2 = dy2.shape
        N1 = z1.shape[1]
        need = ctx.needs_input_grad
        acc2, db2 = _bias_grad_buffer(b2, need[4], N2, dy2.device)
        if acc2 is not None:
            _check(l.dl4j_bias_act_bwd(_ptr(dy2), None, None, _ptr(acc2), M, N2, 0, _DT[dy2.dtype], _stream()), "dl4j_bias_act_bwd")
        dW2 = _weight_grad(W2, y1, dy2) if need[3] else None
        # dz1 = (dy2 @ W2^T) * act'(z1): one GEMM
        dz1 = gemm_raw(dy2, W2_lp.t(), residual=z1, res_act=ctx.act)
        acc1, db1 = _bias_grad_buffer(b1, need[2], N1, dy2.device)
        if acc1 is not None:
            _check(l.dl4j_bias_act_bwd(_ptr(dz1), None, None, _ptr(acc1), M, N1, 0, _DT[dz1.dtype], _stream()), "dl4j_bias_act_bwd")
        dW1 = _weight_grad(W1, x, dz1) if need[1] else None
        dx = gemm_raw(dz1, W1_lp.t()) if need[0] else None
        if db1 is not None:
            db1 = db1.reshape(b1.shape).to(b1.dtype)
        if db2 is not None:
            db2 = db2.reshape(b2.shape).to(b2.dtype)
        return dx, dW1, db1, dW2, db2, None, None, None


def _lp_weight(W, dtype):
    W_lp = getattr(W, "_lp", None)
    if W_lp is None:
        if W.stride(0) != 1 and W.stride(1) != 1:
            return None
        W_lp = W.detach() if W.dtype == dtype else W.detach().to(dtype)
    return W_lp if W_lp.dtype == dtype else None


def mlp(x, W1, b1, W2, b2, activation):
    """``act(x @ W1 + b1) @ W2 + b2`` with the activation gradient folded into the second layer's data-gradient GEMM; returns None
    when the case is not covered (then the two layers run separately)."""
    if not available() or x.dim() != 2 or x.dtype not in (torch.bfloat16, torch.float16):
        return None
    act = _act_id(activation)
    if act not in (1, 2, 3, 4, 5, 6):
        return None
    W1_lp, W2_lp = _lp_weight(W1, x.dtype), _lp_weight(W2, x.dtype)
    if W1_lp is None or W2_lp is None or W1_lp.shape[1] != W2_lp.shape[0]:
        return None
    if not x.is_contiguous():
        x = x.contiguous()
    for w in (W1_lp, W2_lp):
        if _operand_b(w) is None or _operand_b(w.t()) is None or w.shape[0] % 8 or w.shape[1] % 8:
            return None
    if _operand_a(x) is None:
        return None
    return _MlpFn.apply(x, W1, b1, W2, b2, act, W1_lp, W2_lp)


class _LinearFn(torch.autograd.Function):
    """y = act(x @ W + b).  ``W`` is the fp32 (or bf16) leaf, ``W_lp`` its low-precision shadow used
    by the GEMMs.  When ``W`` is a leaf with a preallocated row-major-transposed ``.grad`` view (the
    DL4J 'f' layout inside the flat gradient buffer), the weight gradient is accumulated straight
    into it by the GEMM epilogue (split-K vector reductions) and ``None`` is returned for it."""

    @staticmethod
    def forward(ctx, x, W, b, act, W_lp):
        need_z = act in (2, 3, 4, 5, 6)
        z = torch.empty((x.shape[0], W_lp.shape[1]), dtype=x.dtype, device=x.device) if need_z and any(ctx.needs_input_grad) else None
        W = getattr(W, "_master", W)          # accumulate weight/bias gradients straight into the fp32 masters
        # the forward GEMM takes the bias in the operand format when there is one (shadow of the master): it is then added
        # by one extra tensor-core step instead of a per-element broadcast in the epilogue
        b_fwd = None
        if b is not None:
            b_fwd = b if b.dtype == x.dtype else getattr(b, "_lp", None)
            if b_fwd is not None:
                b_fwd = b_fwd.detach()
        b = getattr(b, "_master", b) if b is not None else None
        if b_fwd is None:
            b_fwd = b
        y = gemm_raw(x, W_lp, bias=None if b_fwd is None else b_fwd.reshape(-1), act=act, aux=z)
        ctx.act = act
        ctx.has_bias = b is not None
        ctx.W_ref = W
        ctx.b_ref = b
        ctx.save_for_backward(x, W_lp, z if z is not None else (y if act == 1 else None))
        return y

    @staticmethod
    def backward(ctx, dy):
        x, W_lp, saved = ctx.saved_tensors
        act = ctx.act
        l = require()
        if not dy.is_contiguous():
            dy = dy.contiguous()
        M, N = dy.shape
        W, b = ctx.W_ref, ctx.b_ref
        # ---- dz and bias gradient
        db = None
        b_acc = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            if b.is_leaf and b.grad is not None and b.grad.dtype == torch.float32 and b.grad.is_contiguous():
                b_acc = b.grad
            else:
                b_acc = torch.zeros(N, dtype=torch.float32, device=dy.device)
                db = b_acc
        if act != 0:
            dz = torch.empty_like(dy)
            zz = saved
            if zz is None:
                raise RuntimeError("linear backward: activation input was not saved")
            rc = l.dl4j_bias_act_bwd(_ptr(dy), _ptr(zz), _ptr(dz), _ptr(b_acc), M, N, 1 if act == 1 else act, _DT[dy.dtype], _stream())
            _check(rc, "dl4j_bias_act_bwd")
        else:
            dz = dy
            if b_acc is not None:
                rc = l.dl4j_bias_act_bwd(_ptr(dy), None, None, _ptr(b_acc), M, N, 0, _DT[dy.dtype], _stream())
                _check(rc, "dl4j_bias_act_bwd")
        if db is not None:
            db = db.reshape(b.shape).to(b.dtype)
        # ---- data gradient: dx = dz @ W^T
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm_raw(dz, W_lp.t())
        # ---- weight gradient: dW^T [nOut, nIn] = dz^T @ x
        dW = None
        if ctx.needs_input_grad[1]:
            nIn = x.shape[1]
            tiles = ((N + 127) // 128) * ((nIn + 255) // 256)
            splits = _wgrad_splits(tiles, M)
            g = W.grad if (W.is_leaf and W.grad is not None) else None
            if g is not None and g.dim() == 4 and g.shape[2] == 1 and g.shape[3] == 1 and g.is_contiguous():
                g = g.view(g.shape[0], g.shape[1]).t()      # 1x1 convolution kernel [nOut, nIn, 1, 1]: same memory as an 'f' dense weight
            if g is not None and g.dtype == torch.float32 and g.dim() == 2 and g.stride(0) == 1 and g.stride(1) == nIn \
                    and g.data_ptr() % 16 == 0 and nIn % 4 == 0:
                gemm_raw(dz.t(), x, out=g.t(), atomic=True, splits=splits)
            elif g is not None and g.dtype == torch.float32 and g.dim() == 2 and g.is_contiguous() and g.data_ptr() % 16 == 0 \
                    and N % 4 == 0:
                # row-major [nIn, nOut] master (SameDiff variables): dW = x^T dz accumulated in place
                tiles2 = ((nIn + 127) // 128) * ((N + 255) // 256)
                gemm_raw(x.t(), dz, out=g, atomic=True, splits=_wgrad_splits(tiles2, M))
            else:
                dWt = gemm_raw(dz.t(), x, out_dtype=torch.float32, atomic=True, splits=splits)
                dW = dWt.reshape(W.shape).to(W.dtype) if W.dim() == 4 else dWt.t().to(W.dtype)
        return dx, dW, db, None, None


def linear(x, W, b, activation):
    """Fused linear on the tcgen05 GEMM; returns None when the case is not covered."""
    if not available() or x.dim() != 2:
        return None
    act = _act_id(activation)
    if act is None:
        return None
    W_lp = getattr(W, "_lp", None)
    if W_lp is None:
        W_lp = W.detach() if W.dtype == x.dtype else W.detach().to(x.dtype)
        if W.stride(0) != 1 and W.stride(1) != 1:
            return None
    if W_lp.dtype != x.dtype:
        return None
    if not x.is_contiguous():
        x = x.contiguous()
    if ((W.shape[1] % 8) or (x.shape[1] % 8)) and _PAD_ODD_WIDTHS and x.shape[0] >= 256:
        return _linear_padded(x, W, b, act)
    if _operand_a(x) is None or _operand_b(W_lp) is None or _operand_b(W_lp.t()) is None:
        return None
    # wgrad needs x as an MN-major operand: row stride multiple of 8 elements, and dz^T likewise
    if (W_lp.shape[1] % 8) or (x.shape[1] % 8):
        return None
    return _LinearFn.apply(x, W, b, act, W_lp)


def _linear_padded(x, W, b, act):
    """Layer widths that are not multiples of 8 (a 77-symbol alphabet, ten classes): the operands are zero-padded to the next
    multiple with differentiable ops and the fused path runs on the padded problem; the padding columns produce zeros that the
    final slice drops, and their gradients vanish in the slice's backward."""
    import torch.nn.functional as F
    K, N = x.shape[1], W.shape[1]
    Kp, Np = (K + 7) // 8 * 8, (N + 7) // 8 * 8
    xp = F.pad(x, (0, Kp - K)) if Kp != K else x
    Wp = F.pad(W, (0, Np - N, 0, Kp - K))                    # [Kp, Np], row-major copy in the parameter's precision
    bp = None if b is None else F.pad(b.reshape(-1), (0, Np - N))
    Wp_lp = Wp.detach().to(x.dtype)
    if _operand_a(xp) is None or _operand_b(Wp_lp) is None or _operand_b(Wp_lp.t()) is None:
        return None
    y = _LinearFn.apply(xp, Wp, bp, act, Wp_lp)
    return y[:, :N] if Np != N else y


_PAD_ODD_WIDTHS = os.environ.get("DL4J_PAD_ODD_WIDTHS", "1") != "0"


# =========================================================================== layer norm
_LN_ONE_PASS = os.environ.get("DL4J_LN_BWD_ONEPASS", "0") == "1"


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gain, bias, eps, res=None):
        l = require()
        shp = x.shape
        C = shp[-1]
        x2 = x.reshape(-1, C)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        gain = getattr(gain, "_master", gain)
        bias = getattr(bias, "_master", bias) if bias is not None else None
        g32 = gain.detach().float().contiguous().reshape(-1)
        b32 = bias.detach().float().contiguous().reshape(-1) if bias is not None else None
        r2 = s2 = None
        if res is not None:
            # y = LN(x + res): the kernel adds the residual while loading and writes the sum once (kept for the backward)
            r2 = res.reshape(-1, C)
            if not r2.is_contiguous():
                r2 = r2.contiguous()
            s2 = torch.empty_like(x2)
        rc = l.dl4j_layer_norm_fwd(_ptr(x2), _ptr(r2), _ptr(g32), _ptr(b32), _ptr(y), _ptr(s2), _ptr(mean), _ptr(rstd), rows, C,
                                   float(eps), _DT[x.dtype], _stream())
        _check(rc, "dl4j_layer_norm_fwd")
        ctx.has_res = res is not None
        ctx.save_for_backward(x2 if s2 is None else s2, g32, mean, rstd)
        ctx.refs = (gain, bias)
        ctx.shape = shp
        return y.reshape(shp)

    @staticmethod
    def backward(ctx, dy):
        l = require()
        x2, g32, mean, rstd = ctx.saved_tensors
        gain, bias = ctx.refs
        rows, C = x2.shape
        dy2 = dy.reshape(rows, C)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = torch.empty_like(x2)

        def acc_for(p):
            if p is None:
                return None, None
            if p.is_leaf and p.grad is not None and p.grad.dtype == torch.float32 and p.grad.is_contiguous():
                return p.grad, None
            t = torch.zeros(C, dtype=torch.float32, device=dy.device)
            return t, t
        gacc, gret = acc_for(gain)
        bacc, bret = acc_for(bias)
        if _LN_ONE_PASS and C <= 1024 and C % 8 == 0 and all(t is None or t.data_ptr() % 16 == 0 for t in (dy2, x2, dx, g32)):
            # one kernel: dx and the per-block partial sums of dgain / dbias from a single read of dy and x, summed in block order
            if not hasattr(l.dl4j_layer_norm_bwd_noalloc, "_typed"):
                vp = ctypes.c_void_p
                l.dl4j_layer_norm_bwd_noalloc.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                                                          ctypes.c_int, vp]
                l.dl4j_layer_norm_bwd_noalloc.restype = ctypes.c_int
                l.dl4j_layer_norm_bwd_noalloc._typed = True
            rc = l.dl4j_layer_norm_bwd_noalloc(_ptr(dy2), _ptr(x2), _ptr(g32), _ptr(mean), _ptr(rstd), _ptr(dx), _ptr(gacc), _ptr(bacc),
                                               rows, C, _DT[x2.dtype], 1, _stream())
            _check(rc, "dl4j_layer_norm_bwd_noalloc")
        else:
            rc = l.dl4j_layer_norm_bwd(_ptr(dy2), _ptr(x2), _ptr(g32), _ptr(mean), _ptr(rstd), _ptr(dx), _ptr(gacc), _ptr(bacc),
                                       rows, C, _DT[x2.dtype], _stream())
            _check(rc, "dl4j_layer_norm_bwd")
        if gret is not None:
            gret = gret.reshape(gain.shape).to(gain.dtype)
        if bret is not None:
            bret = bret.reshape(bias.shape).to(bias.dtype)
        dx = dx.reshape(ctx.shape)
        return dx, gret, bret, None, (dx if ctx.has_res else None)


def layer_norm(x, gain, bias, eps, residual=None):
    """LN(x) or, with ``residual`` (same shape and dtype as x), LN(x + residual) in one pass."""
    C = x.shape[-1]
    if not available() or C % 8 != 0 or C > 1024 or x.dtype not in _DT:
        return None
    if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype):
        return None
    return _LayerNormFn.apply(x, gain, bias, eps, residual)


# =========================================================================== softmax cross entropy
class _SoftmaxXentFn(torch.autograd.Function):
    """Per-row loss; the forward stores only (loss, log-sum-exp, label mass) and the backward writes the gradient already
    multiplied by the upstream per-row scale, so neither pass materialises an unscaled gradient."""

    @staticmethod
    def forward(ctx, logits, labels, sparse):
        l = require()
        if logits.stride(1) != 1:
            logits = logits.contiguous()
        rows, C = logits.shape
        loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        stats = torch.empty((2, rows), dtype=torch.float32, device=logits.device)
        if sparse:
            idx, lab = labels.reshape(-1).to(torch.int64).contiguous(), None
        else:
            idx, lab = None, labels.to(logits.dtype).contiguous()
        rc = l.dl4j_softmax_xent_fwd(_ptr(logits), _ptr(lab), _ptr(idx), _ptr(loss), _ptr(stats[0]), _ptr(stats[1]), rows, C,
                                     logits.stride(0), -100, _DT[logits.dtype], _stream())
        _check(rc, "dl4j_softmax_xent_fwd")
        ctx.save_for_backward(logits, stats, *([idx] if sparse else [lab]))
        ctx.sparse = sparse
        return loss

    @staticmethod
    def backward(ctx, dloss):
        l = require()
        logits, stats, lab_or_idx = ctx.saved_tensors
        rows, C = logits.shape
        grad = torch.empty((rows, C), dtype=logits.dtype, device=logits.device)
        d = dloss.reshape(-1).float().contiguous()
        idx, lab = (lab_or_idx, None) if ctx.sparse else (None, lab_or_idx)
        rc = l.dl4j_softmax_xent_bwd(_ptr(logits), _ptr(lab), _ptr(idx), _ptr(stats[0]), _ptr(stats[1]), _ptr(d), _ptr(grad), rows, C,
                                     logits.stride(0), grad.stride(0), -100, _DT[logits.dtype], _stream())
        _check(rc, "dl4j_softmax_xent_bwd")
        return grad, None, None


def softmax_xent(logits, labels, sparse):
    if not available() or logits.dim() != 2 or logits.dtype not in _DT:
        return None
    return _SoftmaxXentFn.apply(logits, labels, bool(sparse))


# =========================================================================== row gather (embedding lookup)
class _GatherRowsFn(torch.autograd.Function):
    """``table[idx]`` along dim 0.  The gradient is scattered with fp32 vector reductions: straight into the table's
    preallocated fp32 gradient when it has one (nothing is returned for the table then), else into a fresh fp32 buffer."""

    @staticmethod
    def forward(ctx, table, idx):
        ctx.table_ref = getattr(table, "_master", table)
        ctx.table_dtype, ctx.V = table.dtype, table.shape[0]
        ctx.save_for_backward(idx)
        return torch.index_select(table.detach(), 0, idx)

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        l = require()
        tbl = ctx.table_ref
        if dy.stride(1) != 1 or dy.stride(0) % 8 or dy.data_ptr() % 16:
            dy = dy.contiguous()
        C = dy.shape[1]
        g = tbl.grad if (tbl.is_leaf and tbl.grad is not None) else None
        direct = g is not None and g.dtype == torch.float32 and g.is_contiguous() and g.data_ptr() % 16 == 0
        out = g if direct else torch.zeros((ctx.V, C), dtype=torch.float32, device=dy.device)
        rc = l.dl4j_scatter_add_rows(_ptr(dy), _ptr(idx), _ptr(out), idx.numel(), C, dy.stride(0), ctx.V, _DT[dy.dtype], _stream())
        _check(rc, "dl4j_scatter_add_rows")
        return (None if direct else out.to(ctx.table_dtype)), None


def gather_rows(table, idx):
    """Differentiable ``table[idx]`` (2-D table, 1-D int64 indices) or None when the case is not covered."""
    if not available() or table.dim() != 2 or table.dtype not in _DT or table.shape[1] % 8 or not table.is_contiguous():
        return None
    if not (torch.is_grad_enabled() and table.requires_grad):
        return None
    return _GatherRowsFn.apply(table, idx.reshape(-1).to(torch.int64).contiguous())


# =========================================================================== LSTM cell
class _LstmCellFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, z, c_prev):
        l = require()
        mb, n4 = z.shape
        n = n4 // 4
        z = z.contiguous()
        c_prev = c_prev.contiguous()
        h = torch.empty((mb, n), dtype=z.dtype, device=z.device)
        c = torch.empty((mb, n), dtype=torch.float32, device=z.device)
        need = any(ctx.needs_input_grad)
        gates = torch.empty_like(z) if need else None
        rc = l.dl4j_lstm_cell_fwd(_ptr(z), _ptr(c_prev), _ptr(h), _ptr(c), _ptr(gates), mb, n, _DT[z.dtype], _stream())
        _check(rc, "dl4j_lstm_cell_fwd")
        ctx.save_for_backward(gates, c, c_prev)
        return h, c

    @staticmethod
    def backward(ctx, dh, dc):
        l = require()
        gates, c, c_prev = ctx.saved_tensors
        mb, n = c.shape
        dz = torch.empty_like(gates)
        dc_prev = torch.empty_like(c)
        dh = dh.contiguous() if dh is not None else None
        dc = dc.contiguous().float() if dc is not None else None
        rc = l.dl4j_lstm_cell_bwd(_ptr(dh), _ptr(dc), _ptr(gates), _ptr(c), _ptr(c_prev), _ptr(dz), _ptr(dc_prev), mb, n,
                                  _DT[gates.dtype], _stream())
        _check(rc, "dl4j_lstm_cell_bwd")
        return dz, dc_prev


def lstm_cell(z, c_prev):
    if not available() or z.dtype not in _DT or c_prev.dtype != torch.float32:
        return None
    return _LstmCellFn.apply(z, c_prev)


class _LstmSeqFn(torch.autograd.Function):
    """Whole-sequence LSTM layer: forward is one persistent cooperative kernel (recurrent weights resident in
    shared memory, tcgen05 MMAs per step, grid-wide step barrier); backward walks the steps with the fused
    cell-gradient kernel plus one small GEMM per step and finishes with a single large weight-gradient GEMM.
    Gate order and math: libnd4j ops/declarable/helpers/impl/lstmLayer.cpp, LSTMHelpers.java."""

    _scratch = {}
    PERSISTENT_BACKWARD = True       # False: per-step cell-gradient kernel + GEMM (kept as the cross-check path)

    @staticmethod
    def forward(ctx, zx, rw, h0, c0, reverse, rw_lp):
        l = require()
        T, mb, n4 = zx.shape
        n = n4 // 4
        zx = zx.contiguous()
        rw_t = rw_lp.t().contiguous()              # [4n, n]; a no-op for the 'f'-ordered parameter view
        ctx.rw_dtype = rw.dtype
        dev = zx.device
        h_all = torch.empty((T + 1, mb, n), dtype=torch.bfloat16, device=dev)
        h_all[0].copy_(h0)
        cs = torch.empty((T, mb, n), dtype=torch.float32, device=dev)
        gates = torch.empty((T, mb, n4), dtype=torch.bfloat16, device=dev)
        counter = _LstmSeqFn._scratch.get(dev)
        if counter is None:
            counter = _LstmSeqFn._scratch[dev] = torch.zeros(64, dtype=torch.int32, device=dev)
        c0 = c0.contiguous()
        rc = l.dl4j_lstm_seq_fwd(_ptr(zx), _ptr(rw_t), _ptr(h_all), _ptr(c0), _ptr(cs), _ptr(gates), T, mb, n, int(bool(reverse)),
                                 _ptr(counter), _stream())
        _check(rc, "dl4j_lstm_seq_fwd")
        ctx.reverse = bool(reverse)
        ctx.save_for_backward(rw_t, h_all, cs, gates, c0)
        out = h_all[1:].flip(0) if reverse else h_all[1:]
        t_last = 0 if reverse else T - 1
        return out, h_all[T], cs[t_last]

    @staticmethod
    def backward(ctx, dout, dh_last, dc_last):
        l = require()
        rw_t, h_all, cs, gates, c0 = ctx.saved_tensors
        T, mb, n = cs.shape
        rev = ctx.reverse
        dout = dout.contiguous() if dout is not None else torch.zeros((T, mb, n), dtype=torch.bfloat16, device=cs.device)
        dzx = torch.empty_like(gates)
        dc = dc_last.contiguous().float() if dc_last is not None else None
        dh_rec = dh_last.to(torch.bfloat16) if dh_last is not None else None
        dt = _DT[gates.dtype]
        stream = _stream()
        persistent = _LstmSeqFn.PERSISTENT_BACKWARD and dout.dtype == torch.bfloat16
        if persistent:
            # every step of the gradient recursion in one cooperative kernel; weights as [n, 4n] row-major
            if dh_rec is not None:
                dout = dout.clone()
                dout[0 if rev else T - 1] += dh_rec
            rwt = transpose16(rw_t)
            need_h0, need_c0 = ctx.needs_input_grad[2], ctx.needs_input_grad[3]
            dh0 = torch.empty((mb, n), dtype=torch.bfloat16, device=cs.device) if need_h0 else None
            dc0 = torch.empty_like(c0) if need_c0 else None
            counter = _LstmSeqFn._scratch[cs.device]
            rc = l.dl4j_lstm_seq_bwd(_ptr(dout), _ptr(gates), _ptr(cs), _ptr(c0), _ptr(rwt), _ptr(dzx), _ptr(dc), _ptr(dh0), _ptr(dc0),
                                     T, mb, n, int(rev), _ptr(counter), stream)
            _check(rc, "dl4j_lstm_seq_bwd")
            dh_rec, dc = dh0, dc0
        dc_bufs = (torch.empty_like(c0), torch.empty_like(c0))
        for s in (range(T - 1, -1, -1) if not persistent else ()):
            t = T - 1 - s if rev else s
            if s == T - 1:
                dh = dout[t] if dh_rec is None else dout[t] + dh_rec
            else:
                dh = dh_rec
            if s > 0:
                tp = t + 1 if rev else t - 1
                c_prev = cs[tp]
            else:
                c_prev = c0
            dc_new = dc_bufs[s & 1]
            rc = l.dl4j_lstm_cell_bwd(_ptr(dh), _ptr(dc), _ptr(gates[t]), _ptr(cs[t]), _ptr(c_prev), _ptr(dzx[t]), _ptr(dc_new), mb, n,
                                      dt, stream)
            _check(rc, "dl4j_lstm_cell_bwd")
            dc = dc_new
            if s > 0:
                tn = t + 1 if rev else t - 1           # time index processed by step s - 1
                dh_rec = torch.addmm(dout[tn], dzx[t], rw_t)
            else:
                dh_rec = torch.mm(dzx[t], rw_t) if ctx.needs_input_grad[2] else None
        drw = None
        if ctx.needs_input_grad[1]:
            h_prev = h_all[:T].flip(0) if rev else h_all[:T]      # hidden state entering each time index
            a, b = dzx.reshape(T * mb, 4 * n).t(), h_prev.reshape(T * mb, n)
            if ctx.rw_dtype == torch.float32 and _operand_a(a) is not None and _operand_b(b) is not None:
                drw_t = gemm_raw(a, b, out_dtype=torch.float32)
            else:
                drw_t = torch.mm(a, b).to(ctx.rw_dtype)
            drw = drw_t.t()
        return dzx, drw, dh_rec, (dc if ctx.needs_input_grad[3] else None), None, None


def transpose16(m):
    """Dense 2-D bf16 / fp16 matrix -> its transpose as a new dense matrix (tiled kernel; falls back to the strided copy)."""
    if m.dim() == 2 and m.is_contiguous() and m.is_cuda and m.element_size() == 2 and m.shape[0] % 2 == 0 and m.shape[1] % 2 == 0:
        out = torch.empty((m.shape[1], m.shape[0]), dtype=m.dtype, device=m.device)
        rc = require().dl4j_transpose16(_ptr(m), _ptr(out), m.shape[0], m.shape[1], _stream())
        _check(rc, "dl4j_transpose16")
        return out
    return m.t().contiguous()


def lstm_seq_supported(zx, n, mb):
    return (available() and zx.is_cuda and zx.dtype == torch.bfloat16 and n % 64 == 0 and 64 <= n <= 1280 and 1 <= mb <= 128)


def lstm_seq(zx, rw, h0, c0, reverse=False):
    """``zx`` [T, mb, 4n] bf16 input pre-activations, ``rw`` [n, 4n] recurrent weights.  Returns (h for every
    time index [T, mb, n], last h, last c)."""
    rw_lp = getattr(rw, "_lp", None)
    if rw_lp is None or rw_lp.dtype != zx.dtype:
        rw_lp = rw.detach() if rw.dtype == zx.dtype else rw.detach().to(zx.dtype)
    return _LstmSeqFn.apply(zx, rw, h0, c0, reverse, rw_lp)


class _ConvWeightFn(torch.autograd.Function):
    """fp32 [O, I, kH, kW] convolution kernel -> bf16 channels-last view for the tensor-core convolution kernels (one cast +
    relayout pass); the channels-last weight gradient is added straight into the fp32 gradient buffer of the parameter."""

    @staticmethod
    def forward(ctx, W):
        l = require()
        O, I, kH, kW = W.shape
        buf = torch.empty((O, kH, kW, I), dtype=torch.bfloat16, device=W.device)
        Wm = getattr(W, "_master", W)
        rc = l.dl4j_conv_weight_to_cl(_ptr(Wm.detach().contiguous()), _ptr(buf), O, I, kH * kW, _stream())
        _check(rc, "dl4j_conv_weight_to_cl")
        ctx.W_ref = Wm
        return buf.permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, dW):
        l = require()
        W = ctx.W_ref
        O, I, kH, kW = W.shape
        g_cl = dW.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        tgt = W.grad if (W.is_leaf and W.grad is not None and W.grad.dtype == torch.float32 and W.grad.is_contiguous()) else None
        out = tgt if tgt is not None else torch.zeros(W.shape, dtype=torch.float32, device=W.device)
        rc = l.dl4j_conv_wgrad_from_cl(_ptr(g_cl), _ptr(out), O, I, kH * kW, _stream())
        _check(rc, "dl4j_conv_wgrad_from_cl")
        return None if tgt is not None else out.to(W.dtype)


def _conv_sigs(l):
    if getattr(l, "_conv_typed", False):
        return
    vp, i32 = ctypes.c_void_p, ctypes.c_int
    l.dl4j_conv2d.argtypes = [i32, vp, vp, vp, vp] + [i32] * 17 + [vp]
    l.dl4j_conv2d.restype = i32
    l.dl4j_conv2d_wgrad.argtypes = [vp, vp, vp] + [i32] * 15 + [vp]
    l.dl4j_conv2d_wgrad.restype = i32
    l.dl4j_conv_wgrad_f32_from_cl.argtypes = [vp, vp, i32, i32, i32, vp]
    l.dl4j_conv_wgrad_f32_from_cl.restype = i32
    l._conv_typed = True


class _Conv2dFn(torch.autograd.Function):
    """Stride-1 2-D convolution on the tcgen05 implicit-GEMM kernels (``csrc/conv_tcgen05.cu``): forward, data gradient
    and weight gradient.  ``x`` is a channels-last 16-bit activation [N, Cin, H, W].  ``W`` is either the fp32 parameter
    [Cout, Cin, kH, kW] (it is cast and laid out channels-last here, and its gradient is added straight into the
    parameter's fp32 gradient buffer when it has one) or an already channels-last 16-bit kernel (its gradient is returned).
    ``fuse_w``: few-channel stem form, see ``dl4j_conv2d``."""

    @staticmethod
    def forward(ctx, x, W, bias, pad, dil, fuse_w, path=0):
        l = require()
        _conv_sigs(l)
        x = _dense_cl(x)
        N, Cin, H, Wd = x.shape
        Wm = getattr(W, "_master", W)
        Cout, _, kH, kW = Wm.shape
        if Wm.dtype == torch.float32:
            w_cl = torch.empty((Cout, kH, kW, Cin), dtype=x.dtype, device=x.device)
            if x.dtype == torch.bfloat16 and Wm.is_contiguous():
                rc = l.dl4j_conv_weight_to_cl(_ptr(Wm.detach()), _ptr(w_cl), Cout, Cin, kH * kW, _stream())
                _check(rc, "dl4j_conv_weight_to_cl")
            else:
                w_cl.copy_(Wm.detach().permute(0, 2, 3, 1))
            ctx.master = Wm
        else:
            w_cl = W.detach().permute(0, 2, 3, 1).contiguous()
            ctx.master = None
        OH = H + 2 * pad[0] - (kH - 1) * dil[0]
        OW = Wd + 2 * pad[1] - (kW - 1) * dil[1]
        y = torch.empty((N, OH, OW, Cout), dtype=x.dtype, device=x.device)
        b = None
        if bias is not None:
            b = bias.detach().reshape(-1)
            b = b if b.dtype in (torch.float32, x.dtype) else b.float()
            b = b.contiguous()
        ctx.geom = (N, H, Wd, Cin, OH, OW, Cout, kH, kW, int(pad[0]), int(pad[1]), int(dil[0]), int(dil[1]))
        ctx.fuse_w = int(bool(fuse_w))
        ctx.path = int(path)          # 0 automatic, 2 per-tap kernel, 4 halo kernel (tests)
        rc = l.dl4j_conv2d(0, _ptr(x), _ptr(w_cl), _ptr(y), _ptr(b), *ctx.geom, _DT[x.dtype],
                           1 if (b is not None and b.dtype == torch.float32) else 0, 0, ctx.fuse_w | ctx.path, _stream())
        _check(rc, "dl4j_conv2d")
        ctx.has_bias = bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        ctx.bias_shape = tuple(bias.shape) if bias is not None else None
        ctx.w_dtype = W.dtype
        ctx.save_for_backward(x, w_cl)
        return y.permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, dy):
        l = require()
        x, w_cl = ctx.saved_tensors
        N, H, Wd, Cin, OH, OW, Cout, kH, kW, ph, pw, dh, dw_ = ctx.geom
        dy = _dense_cl(dy)
        if dy.dtype != x.dtype:
            dy = dy.to(x.dtype)
        dx = dW = db = None
        if ctx.needs_input_grad[0]:
            dxb = torch.empty((N, H, Wd, Cin), dtype=x.dtype, device=x.device)
            rc = l.dl4j_conv2d(1, _ptr(dy), _ptr(w_cl), _ptr(dxb), None, *ctx.geom, _DT[x.dtype], 0, 0, ctx.path, _stream())
            _check(rc, "dl4j_conv2d")
            dx = dxb.permute(0, 3, 1, 2)
        if ctx.needs_input_grad[1] or ctx.master is not None:
            g_cl = torch.zeros((Cout, kH, kW, Cin), dtype=torch.float32, device=x.device)
            rc = l.dl4j_conv2d_wgrad(_ptr(dy), _ptr(x), _ptr(g_cl), *ctx.geom, _DT[x.dtype], ctx.fuse_w, _stream())
            _check(rc, "dl4j_conv2d_wgrad")
            Wm = ctx.master
            if Wm is not None:
                tgt = Wm.grad if (Wm.is_leaf and Wm.grad is not None and Wm.grad.dtype == torch.float32 and Wm.grad.is_contiguous()) else None
                out = tgt if tgt is not None else torch.zeros(Wm.shape, dtype=torch.float32, device=x.device)
                rc = l.dl4j_conv_wgrad_f32_from_cl(_ptr(g_cl), _ptr(out), Cout, Cin, kH * kW, _stream())
                _check(rc, "dl4j_conv_wgrad_f32_from_cl")
                dW = None if tgt is not None else out.to(ctx.w_dtype)
            else:
                dW = g_cl.permute(0, 3, 1, 2).to(ctx.w_dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.float().sum((0, 2, 3)).reshape(ctx.bias_shape).to(ctx.bias_dtype)
        return dx, dW, db, None, None, None, None


def conv2d(x, W, bias, pad, dil, fuse_w=False, path=None):
    """Stride-1 convolution on the native implicit-GEMM kernels, or None when the case is not covered (the caller then
    uses the library path): 16-bit CUDA activation, channel counts multiples of 8, non-negative output size."""
    if not (available() and x.is_cuda and x.dim() == 4 and x.dtype in (torch.bfloat16, torch.float16)):
        return None
    Wm = getattr(W, "_master", W)
    if Wm.dim() != 4 or Wm.shape[1] != x.shape[1] or x.shape[1] % 8 or Wm.shape[0] % 8:
        return None
    if Wm.dtype != torch.float32 and Wm.dtype != x.dtype:
        return None
    kH, kW = Wm.shape[2], Wm.shape[3]
    if kH * kW > 64:
        return None
    if x.shape[2] + 2 * pad[0] - (kH - 1) * dil[0] < 1 or x.shape[3] + 2 * pad[1] - (kW - 1) * dil[1] < 1:
        return None
    if pad[0] < 0 or pad[1] < 0 or pad[0] > 255 or pad[1] > 255:
        return None
    if fuse_w and (pad[1] != 0 or dil[1] != 1 or kW * x.shape[1] > 64):
        fuse_w = False
    return _Conv2dFn.apply(x, W, bias, (int(pad[0]), int(pad[1])), (int(dil[0]), int(dil[1])), bool(fuse_w),
                           {None: 0, "tap": 2, "halo": 4}[path])


def conv_weight_cl(W):
    """bf16 channels-last version of an fp32 convolution kernel parameter, or None when not applicable."""
    if not (available() and W.is_cuda and W.dim() == 4 and W.dtype == torch.float32 and W.is_contiguous()):
        return None
    return _ConvWeightFn.apply(W)


class _SubsampleFn(torch.autograd.Function):
    """x[:, :, ::sH, ::sW] of a channels-last bf16 activation as one gather kernel; the gradient is one scatter-with-zeros."""

    @staticmethod
    def forward(ctx, x, sH, sW):
        l = require()
        x = _dense_cl(x)
        N, C, H, W = x.shape
        OH, OW = (H + sH - 1) // sH, (W + sW - 1) // sW
        y = torch.empty((N, C, OH, OW), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
        ctx.shape = (N, H, W, C, OH, OW, 1, 1, sH, sW, 0, 0)
        rc = l.dl4j_subsample(_ptr(x), _ptr(y), (ctypes.c_int * 12)(*ctx.shape), 0, _stream())
        _check(rc, "dl4j_subsample")
        return y

    @staticmethod
    def backward(ctx, dy):
        l = require()
        N, H, W, C = ctx.shape[:4]
        dy = _dense_cl(dy)
        dx = torch.empty((N, C, H, W), dtype=dy.dtype, device=dy.device, memory_format=torch.channels_last)
        rc = l.dl4j_subsample(_ptr(dy), _ptr(dx), (ctypes.c_int * 12)(*ctx.shape), 1, _stream())
        _check(rc, "dl4j_subsample")
        return dx, None, None


def stem_space_to_depth(x, pad, Hs, Ws, CP):
    """2x2 space-to-depth view of the zero-padded input ``x`` [N, C, H, W] (16-bit, any strides, no gradient) as a channels-last
    tensor [N, CP, Hs, Ws] with channel (bh * 2 + bw) * C + c; one pass instead of pad / reshape / permute / pad / contiguous.
    Returns None when the case is not covered."""
    if not available() or x.requires_grad or x.dtype not in (torch.bfloat16, torch.float16) or CP not in (8, 16, 32):
        return None
    N, C, H, W = x.shape
    if 4 * C > CP:
        return None
    l = require()
    if not hasattr(l.dl4j_stem_space_to_depth, "_typed"):
        vp, i32 = ctypes.c_void_p, ctypes.c_int
        l.dl4j_stem_space_to_depth.argtypes = [vp, vp, i32, i32, i32, i32, ctypes.POINTER(ctypes.c_longlong), i32, i32, i32, i32, i32, vp]
        l.dl4j_stem_space_to_depth.restype = ctypes.c_int
        l.dl4j_stem_space_to_depth._typed = True
    out = torch.empty((N, Hs, Ws, CP), dtype=x.dtype, device=x.device)
    st = (ctypes.c_longlong * 4)(*x.stride())
    rc = l.dl4j_stem_space_to_depth(_ptr(x), _ptr(out), N, C, H, W, st, int(pad[0]), int(pad[1]), Hs, Ws, CP, _stream())
    _check(rc, "dl4j_stem_space_to_depth")
    return out.permute(0, 3, 1, 2)


def conv1x1(x, W, b, stride=(1, 1)):
    """1x1 convolution over a channels-last activation as one tcgen05 GEMM: [N*H*W, Cin] x [Cin, Cout] (forward, data
    gradient and weight gradient all run on the hand-written kernel).  ``W`` is the [Cout, Cin, 1, 1] parameter; returns
    None when the case is not covered."""
    if not available() or not x.is_cuda or x.dim() != 4 or x.dtype not in (torch.bfloat16, torch.float16):
        return None
    Cout, Cin = W.shape[0], W.shape[1]
    if W.dim() != 4 or W.shape[2] != 1 or W.shape[3] != 1 or Cin % 8 or Cout % 8 or x.shape[1] != Cin:
        return None
    W_lp = getattr(W, "_lp", None)
    if W_lp is None or W_lp.dtype != x.dtype:
        W_lp = W.detach() if W.dtype == x.dtype else W.detach().to(x.dtype)
    if not W_lp.is_contiguous() or W_lp.data_ptr() % 16:
        return None
    if stride[0] != 1 or stride[1] != 1:
        x = _SubsampleFn.apply(x, int(stride[0]), int(stride[1])) if x.dtype == torch.bfloat16 else x[:, :, ::stride[0], ::stride[1]]
    x = _dense_cl(x)
    N, _, H, Wd = x.shape
    x2 = x.permute(0, 2, 3, 1).reshape(N * H * Wd, Cin)
    if _operand_a(x2) is None:
        return None
    y2 = _LinearFn.apply(x2, W, b, 0, W_lp.view(Cout, Cin).t())
    return y2.view(N, H, Wd, Cout).permute(0, 3, 1, 2)


class _MaxPoolFn(torch.autograd.Function):
    """Channels-last max pooling; forward keeps one byte per output element (winning window position), backward gathers."""

    @staticmethod
    def forward(ctx, x, k, s, p):
        l = require()
        x = _dense_cl(x)
        N, C, H, W = x.shape
        OH = (H + 2 * p[0] - k[0]) // s[0] + 1
        OW = (W + 2 * p[1] - k[1]) // s[1] + 1
        y = torch.empty((N, C, OH, OW), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
        need = ctx.needs_input_grad[0]
        idx = torch.empty(N * OH * OW * C, dtype=torch.uint8, device=x.device) if need else None
        shape = (ctypes.c_int * 12)(N, H, W, C, OH, OW, k[0], k[1], s[0], s[1], p[0], p[1])
        rc = l.dl4j_maxpool_fwd(_ptr(x), _ptr(y), _ptr(idx), shape, _stream())
        _check(rc, "dl4j_maxpool_fwd")
        ctx.shape = (N, H, W, C, OH, OW, k[0], k[1], s[0], s[1], p[0], p[1])
        ctx.save_for_backward(idx)
        return y

    @staticmethod
    def backward(ctx, dy):
        l = require()
        (idx,) = ctx.saved_tensors
        N, H, W, C = ctx.shape[:4]
        dy = _dense_cl(dy)
        dx = torch.empty((N, C, H, W), dtype=dy.dtype, device=dy.device, memory_format=torch.channels_last)
        shape = (ctypes.c_int * 12)(*ctx.shape)
        rc = l.dl4j_maxpool_bwd(_ptr(dy), _ptr(idx), _ptr(dx), shape, _stream())
        _check(rc, "dl4j_maxpool_bwd")
        return dx, None, None, None


def maxpool2d(x, k, s, p):
    if not (available() and x.is_cuda and x.dim() == 4 and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0):
        return None
    if k[0] * k[1] > 255 or p[0] >= k[0] or p[1] >= k[1] or min(x.shape) == 0:
        return None
    if (x.shape[2] + 2 * p[0] - k[0]) < 0 or (x.shape[3] + 2 * p[1] - k[1]) < 0:
        return None
    return _MaxPoolFn.apply(x, tuple(int(v) for v in k), tuple(int(v) for v in s), tuple(int(v) for v in p))


# =========================================================================== batch norm (+ residual) (+ ReLU)
def _rows_c(x):
    """(rows, C) of a channels-last 4-D or a plain 2-D activation."""
    if x.dim() == 4:
        return x.shape[0] * x.shape[2] * x.shape[3], x.shape[1]
    return x.shape[0], x.shape[1]


def _dense_cl(x):
    """Channels-last dense layout for 4-D tensors, row-major for 2-D ones (copies only when needed)."""
    if x.dim() == 4:
        return x if x.is_contiguous(memory_format=torch.channels_last) else x.contiguous(memory_format=torch.channels_last)
    return x.contiguous()


class _BnActFn(torch.autograd.Function):
    """y = act(batchnorm_train(x) [+ res]) over channels-last bf16 activations; running statistics are updated in place by
    the kernel (``nn/layers/normalization/BatchNormalization.java`` semantics: biased batch variance, decay rule)."""

    @staticmethod
    def forward(ctx, x, res, gamma, beta, run_mean, run_stat, use_log_std, decay, eps, relu, pre_bias=None):
        l = require()
        x = _dense_cl(x)
        res = _dense_cl(res) if res is not None else None
        rows, C = _rows_c(x)
        y = torch.empty_like(x)
        save = torch.empty(2 * C, dtype=torch.float32, device=x.device)
        work = torch.empty(4 * C + 8, dtype=torch.float32, device=x.device)      # [sums | ticket | scale | shift]
        g = gamma.detach().float().contiguous() if gamma is not None else None
        b = beta.detach().float().contiguous() if beta is not None else None
        rc = l.dl4j_bn_fwd_train(_ptr(x), _ptr(res), _ptr(g), _ptr(b), _ptr(run_mean), _ptr(run_stat), int(bool(use_log_std)),
                                 float(decay), float(eps), int(bool(relu)), _ptr(y), _ptr(save), _ptr(save[C:]), _ptr(work),
                                 _ptr(pre_bias), rows, C, _stream())
        _check(rc, "dl4j_bn_fwd_train")
        global LAUNCHES
        LAUNCHES += 2
        ctx.relu, ctx.has_res, ctx.has_affine = bool(relu), res is not None, gamma is not None
        ctx.gb_refs = (gamma, beta)
        ctx.save_for_backward(x, y if (res is not None and relu) else None, save, work)
        return y

    @staticmethod
    def backward(ctx, dy):
        l = require()
        x, y, save, work = ctx.saved_tensors
        rows, C = _rows_c(x)
        dy = _dense_cl(dy)
        dx = torch.empty_like(x)
        dres = torch.empty_like(x) if ctx.has_res else None
        # the kernel adds dgamma / dbeta to what its targets hold: the parameters' preallocated fp32 gradients when they have
        # them (nothing is returned then, so autograd launches no accumulation), else a zeroed scratch that is returned
        def target(p_):
            if p_ is not None and p_.is_leaf and p_.grad is not None and p_.grad.dtype == torch.float32 and p_.grad.is_contiguous() \
                    and p_.grad.numel() == C:
                return p_.grad
            return None
        gamma, beta = ctx.gb_refs
        tg, tb = (target(gamma), target(beta)) if ctx.has_affine else (None, None)
        dgb = None
        if ctx.has_affine and (tg is None or tb is None):
            dgb = torch.zeros(2 * C, dtype=torch.float32, device=x.device)
        pg = tg if tg is not None else (dgb[:C] if dgb is not None else None)
        pb = tb if tb is not None else (dgb[C:] if dgb is not None else None)
        rc = l.dl4j_bn_bwd(_ptr(dy), _ptr(x), _ptr(y), _ptr(save), _ptr(save[C:]), _ptr(work), _ptr(dx), _ptr(dres),
                           _ptr(pg), _ptr(pb), rows, C, int(ctx.relu), _stream())
        _check(rc, "dl4j_bn_bwd")
        global LAUNCHES
        LAUNCHES += 1
        dg = pg.reshape(gamma.shape) if (ctx.has_affine and tg is None and ctx.needs_input_grad[2]) else None
        db = pb.reshape(beta.shape) if (ctx.has_affine and tb is None and ctx.needs_input_grad[3]) else None
        return dx, dres, dg, db, None, None, None, None, None, None, None


def bn_supported(x):
    if not (available() and x.is_cuda and x.dtype == torch.bfloat16 and x.dim() in (2, 4)):
        return False
    rows, C = _rows_c(x)
    return rows > 0 and 8 <= C <= 2048 and (C & (C - 1)) == 0


def bn_act_train(x, res, gamma, beta, run_mean, run_stat, use_log_std, decay, eps, relu, pre_bias=None):
    """Fused training-mode batch norm; ``gamma`` / ``beta`` fp32 [C] (or None), running buffers fp32 [C] updated in place.
    ``pre_bias`` (fp32 [C]) is a bias that the producer left out of ``x``: it only enters the running mean."""
    pb = pre_bias.detach().float().reshape(-1).contiguous() if pre_bias is not None else None
    # gamma / beta go in as they are (any shape with C elements): a reshape would hide a parameter leaf and its gradient slice
    return _BnActFn.apply(x, res, gamma, beta, run_mean, run_stat, use_log_std, decay, eps, relu, pb)


def bn_act_eval(x, res, scale, shift, relu):
    """y = act(x * scale + shift [+ res]) with fp32 per-channel scale / shift (inference statistics folded in)."""
    l = require()
    x = _dense_cl(x)
    res = _dense_cl(res) if res is not None else None
    rows, C = _rows_c(x)
    y = torch.empty_like(x)
    rc = l.dl4j_bn_apply(_ptr(x), _ptr(res), _ptr(scale.float().contiguous()), _ptr(shift.float().contiguous()), int(bool(relu)), _ptr(y),
                         rows, C, _stream())
    _check(rc, "dl4j_bn_apply")
    return y


class _AddReluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        l = require()
        a = _dense_cl(a)
        b = _dense_cl(b)
        if b.stride() != a.stride():
            b = b.contiguous(memory_format=torch.channels_last) if a.dim() == 4 else b.contiguous()
        y = torch.empty_like(a)
        rc = l.dl4j_add_relu(_ptr(a), _ptr(b), _ptr(y), a.numel(), _stream())
        _check(rc, "dl4j_add_relu")
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        g = dy * (y > 0).to(dy.dtype)
        return g, g


def add_relu(a, b):
    if not (available() and a.is_cuda and a.dtype == torch.bfloat16 and a.shape == b.shape and a.numel() % 8 == 0 and a.dim() in (2, 4)):
        return None
    return _AddReluFn.apply(a, b)


def attention(q, k, v, mask, scale, dropout_p=0.0):
    from . import attention_native
    return attention_native.attention(q, k, v, mask, scale, dropout_p)


# =========================================================================== fused updater
_SEG_FMT = "<qqqqqfffiii"     # offset, block_start, block_numel, state_off, shadow_off, l1, l2, wd, kernel_id, hyper, pad
_CHUNK_FMT = "<qii"
_CHUNK = int(os.environ.get("DL4J_UPDATER_CHUNK", "16384"))     # elements per block of the multi-segment updater launch


def _cfg_index(known, cfg):
    """Index of ``cfg`` among the distinct updater configurations seen so far (hyper-parameter sets are per
    configuration, not per state block)."""
    for i, c in enumerate(known):
        if c is cfg or c == cfg:
            return i
    known.append(cfg)
    return len(known) - 1


def _build_tables(upd, shadow_offsets):
    """Static part of the segment / chunk tables for a MultiLayerUpdater."""
    segs = upd.segments(0, 0)
    block_ids = []
    seg_rows, chunks = [], []
    upd._seg_chunk0 = []                 # first chunk of every segment (bucketed gradient exchange addresses chunk ranges)
    for si, (off, numel, st_off, bn, bs, kid, lr, l1, l2, wd, cfg) in enumerate(segs):
        upd._seg_chunk0.append(len(chunks))
        hid = _cfg_index(block_ids, cfg)
        seg_rows.append([off, bs, bn, st_off, shadow_offsets[si] if shadow_offsets is not None else 0, l1, l2, wd, kid, hid, 0])
        o = 0
        while o < numel:
            c = min(_CHUNK, numel - o)
            chunks.append(struct.pack(_CHUNK_FMT, off + o, c, si))
            o += c
    upd._seg_chunk0.append(len(chunks))
    return seg_rows, b"".join(chunks), len(chunks), len(block_ids)


def update_tables(upd, iteration, epoch, shadow_offsets=None):
    """Device chunk/segment tables + this iteration's hyper-parameter table for ``upd``; None if unsupported."""
    cache = getattr(upd, "_native_tables", None)
    if cache is None or cache["shadow"] is not shadow_offsets:
        seg_rows, chunk_bytes, n_chunks, n_hyper = _build_tables(upd, shadow_offsets)
        if n_hyper > 8:
            upd._native_tables = {"unsupported": True, "shadow": shadow_offsets}
            return None
        dev = upd.params.device
        chunks_t = torch.frombuffer(bytearray(chunk_bytes), dtype=torch.uint8).to(dev)
        cache = {"seg_rows": seg_rows, "chunks": chunks_t, "n_chunks": n_chunks, "n_hyper": n_hyper, "shadow": shadow_offsets,
                 "segs_dev": None, "segs_key": None}
        upd._native_tables = cache
    if cache.get("unsupported"):
        return None
    # dynamic part: per-block hyper-parameters and any scheduled regularisation coefficients
    segs = upd.segments(iteration, epoch)
    hyper = np.zeros((8, 8), dtype=np.float32)
    key = []
    seen = []
    for si, (off, numel, st_off, bn, bs, kid, lr, l1, l2, wd, cfg) in enumerate(segs):
        key.append((l1, l2, wd))
        hid = _cfg_index(seen, cfg)
        b1 = getattr(cfg, "beta1", 0.0); b2 = getattr(cfg, "beta2", 0.0); eps = getattr(cfg, "epsilon", 0.0)
        from ..nn.updaters import _eps_t, Nesterovs, AdaMax
        eps_t = 0.0
        if hasattr(cfg, "beta1"):
            eps_t = _eps_t(lr, b1, b2, iteration, eps, with_sqrt=not isinstance(cfg, AdaMax))
        mu = cfg.currentMomentum(iteration, epoch) if isinstance(cfg, Nesterovs) else 0.0
        rho = getattr(cfg, "rmsDecay", getattr(cfg, "rho", 0.0))
        mb1t = 1.0 - b1 ** (iteration + 1) if b1 else 1.0
        hyper[hid] = (lr, b1, b2, eps, eps_t, mb1t, mu, rho)
    key = tuple(key)
    if cache["segs_key"] != key:
        rows = cache["seg_rows"]
        buf = bytearray()
        for r, (l1, l2, wd) in zip(rows, key):
            buf += struct.pack(_SEG_FMT, r[0], r[1], r[2], r[3], r[4], l1, l2, wd, r[8], r[9], 0)
        cache["segs_dev"] = torch.frombuffer(buf, dtype=torch.uint8).to(upd.params.device)
        cache["segs_key"] = key
    cache["hyper"] = hyper
    return cache


def fused_update(upd, iteration, epoch, shadow=None, shadow_offsets=None, grad_scale=1.0, zero_grads=True, residual=None) -> bool:
    """One launch: regularisation + updater + params -= update (+ bf16 shadow refresh, + grad zeroing); with
    ``residual`` the update is accumulated into it instead and the parameters are left untouched."""
    l = require()
    if l is None:
        return False
    cache = update_tables(upd, iteration, epoch, shadow_offsets)
    if cache is None:
        return False
    hyper = cache["hyper"]
    state = upd.state
    hp = hyper.ctypes.data_as(ctypes.c_void_p)
    rc = l.dl4j_fused_update(_ptr(upd.params), _ptr(upd.grads), _ptr(state) if state.numel() else None, _ptr(shadow),
                             _ptr(residual), _ptr(cache["chunks"]), cache["n_chunks"], _ptr(cache["segs_dev"]), hp, cache["n_hyper"],
                             float(grad_scale), 1 if zero_grads else 0, _stream())
    _check(rc, "dl4j_fused_update")
    upd._fused_zeroes_grads = bool(zero_grads)
    return True


def cast_to_bf16(src_f32, dst_bf16):
    l = require()
    rc = l.dl4j_cast_f32_bf16(_ptr(src_f32), _ptr(dst_bf16), src_f32.numel(), _stream())
    _check(rc, "dl4j_cast_f32_bf16")


# =========================================================================== gradient codecs
def threshold_encode(x, tau, capacity=None, msg=None):
    """In-place sparse threshold encode of fp32 ``x`` (residual stays in ``x``); returns the int32 message."""
    l = require()
    n = x.numel()
    capacity = int(capacity if capacity is not None else n)
    if msg is None:
        msg = torch.empty(4 + capacity, dtype=torch.int32, device=x.device)
    rc = l.dl4j_threshold_encode(_ptr(x), n, float(tau), _ptr(msg), capacity, _stream())
    _check(rc, "dl4j_threshold_encode")
    return msg


def threshold_decode(msg, target, scale=1.0, atomics=False, capacity=None):
    l = require()
    capacity = int(capacity if capacity is not None else msg.numel() - 4)
    rc = l.dl4j_threshold_decode(_ptr(msg), capacity, _ptr(target), target.numel(), float(scale), 1 if atomics else 0, _stream())
    _check(rc, "dl4j_threshold_decode")
    return target


def bitmap_encode(x, tau, msg=None):
    l = require()
    n = x.numel()
    if msg is None:
        msg = torch.empty(4 + (n + 15) // 16, dtype=torch.int32, device=x.device)
    rc = l.dl4j_bitmap_encode(_ptr(x), n, float(tau), _ptr(msg), _stream())
    _check(rc, "dl4j_bitmap_encode")
    return msg


def bitmap_decode(msg, target, scale=1.0):
    l = require()
    rc = l.dl4j_bitmap_decode(_ptr(msg), _ptr(target), target.numel(), float(scale), _stream())
    _check(rc, "dl4j_bitmap_decode")
    return target


# =========================================================================== word2vec / t-SNE
def w2v_batch(syn0, syn1, syn1neg, neg_table, target, ng_starter, points, codes, context, alpha, random, ns_rounds, train_words=True):
    """One launch of the skip-gram (``context`` None) or CBOW output-layer update for a batch of examples, in place on the fp32
    tables.  ``target`` / ``ng_starter`` [B], ``points`` / ``codes`` [B, L] (-1 padded) or None, ``context`` [B, W] (-1 padded) or
    None, ``alpha`` fp32 [B] or [1], ``random`` int64 [B] or [1].  Returns False when the case is not covered."""
    l = lib()
    if l is None or not syn0.is_cuda or syn0.dtype != torch.float32 or not syn0.is_contiguous() or syn0.dim() != 2:
        return False
    for t in (syn1, syn1neg):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or t.shape[1] != syn0.shape[1]):
            return False
    dev = syn0.device
    V, D = int(syn0.shape[0]), int(syn0.shape[1])
    if D > 4096:
        return False

    def i32(t):
        return None if t is None else t.to(device=dev, dtype=torch.int32).contiguous()
    target = i32(target.reshape(-1))
    B = int(target.numel())
    if B == 0:
        return True
    ng_starter = i32(ng_starter.reshape(-1)) if ng_starter is not None else None
    L = W = 0
    if points is not None and syn1 is not None:
        points = i32(points.reshape(B, -1))
        codes = codes.reshape(B, -1).to(device=dev, dtype=torch.int8).contiguous()
        L = int(points.shape[1])
    else:
        points = codes = None
    if context is not None:
        context = i32(context.reshape(B, -1))
        W = int(context.shape[1])
    neg_table = i32(neg_table.reshape(-1)) if neg_table is not None and neg_table.numel() else None
    alpha = alpha.to(device=dev, dtype=torch.float32).reshape(-1).contiguous()
    random = random.to(device=dev, dtype=torch.int64).reshape(-1).contiguous()
    if not hasattr(l.dl4j_w2v_batch, "_typed"):
        vp, i32c, i64c = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        l.dl4j_w2v_batch.argtypes = [vp, vp, vp, vp, i64c, vp, vp, vp, vp, vp, vp, i32c, vp, i32c, i32c, i32c, i32c, i32c, i32c, i32c, i32c, vp]
        l.dl4j_w2v_batch.restype = ctypes.c_int
        l.dl4j_w2v_batch._typed = True
    rc = l.dl4j_w2v_batch(_ptr(syn0), _ptr(syn1), _ptr(syn1neg), _ptr(neg_table), 0 if neg_table is None else int(neg_table.numel()),
                          _ptr(target), _ptr(ng_starter), _ptr(points), _ptr(codes), _ptr(context), _ptr(alpha), int(alpha.numel()),
                          _ptr(random), int(random.numel()), B, L, W, D, V, int(ns_rounds), 1 if train_words else 0, _stream())
    _check(rc, "dl4j_w2v_batch")
    return True


def barnes_edge_forces(row_p, col_p, val_p, y):
    """Attractive t-SNE forces over a CSR matrix; ``y`` fp32 [N, D <= 8].  None when the case is not covered."""
    l = lib()
    if l is None or not y.is_cuda or y.dtype != torch.float32 or y.dim() != 2 or y.shape[1] > 8:
        return None
    N, D = int(y.shape[0]), int(y.shape[1])
    row_p = row_p.to(device=y.device, dtype=torch.int32).contiguous()
    col_p = col_p.to(device=y.device, dtype=torch.int32).contiguous()
    val_p = val_p.to(device=y.device, dtype=torch.float32).contiguous()
    y = y.contiguous()
    out = torch.empty_like(y)
    if not hasattr(l.dl4j_barnes_edge_forces, "_typed"):
        vp, i32c = ctypes.c_void_p, ctypes.c_int
        l.dl4j_barnes_edge_forces.argtypes = [vp, vp, vp, vp, vp, i32c, i32c, vp]
        l.dl4j_barnes_edge_forces.restype = ctypes.c_int
        l.dl4j_barnes_edge_forces._typed = True
    rc = l.dl4j_barnes_edge_forces(_ptr(row_p), _ptr(col_p), _ptr(val_p), _ptr(y), _ptr(out), N, D, _stream())
    _check(rc, "dl4j_barnes_edge_forces")
    return out
