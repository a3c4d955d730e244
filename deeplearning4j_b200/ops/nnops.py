"""Neural-network op front door used by layers and SameDiff ops.

Every function has a plain torch implementation (CPU path and numerics oracle).  On a CUDA
device with the native extension loaded, the bf16/fp16 hot shapes are routed to the
hand-written sm_100a kernels in ``ops.native`` (tcgen05 GEMM with fused bias/activation
epilogue, fused layer-norm, fused softmax-cross-entropy, fused LSTM cell, flash attention).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

_FORCE_TORCH = False


def _up(t):
    """At least float32: half / bf16 inputs are computed in fp32, fp64 stays fp64 (gradient checks)."""
    return t if t.dtype in (torch.float32, torch.float64) else t.float()


def set_force_torch(v: bool):
    """Route everything through torch (used to produce the library-only baseline)."""
    global _FORCE_TORCH
    _FORCE_TORCH = bool(v)


def have_fused() -> bool:
    if _FORCE_TORCH or not torch.cuda.is_available():
        return False
    from . import native
    return native.available()


def _native_for(x: torch.Tensor):
    if _FORCE_TORCH or not x.is_cuda:
        return None
    from . import native
    return native if native.available() else None


def linear(x, W, b=None, activation=None, training=False):
    """``act(x @ W + b)`` with ``W`` logical ``[nIn, nOut]`` (DL4J 'f' layout => K-major for the GEMM)."""
    nat = _native_for(x)
    if nat is not None and x.dtype in (torch.bfloat16, torch.float16):
        y = nat.linear(x, W, b, activation)
        if y is not None:
            return y
    if W.dtype != x.dtype:
        W = W.to(x.dtype)
    if b is not None and x.dim() == 2 and b.dtype == x.dtype and b.numel() == W.shape[1]:
        z = torch.addmm(b.reshape(1, -1), x, W)        # bias in the GEMM's epilogue: one launch less per layer
    else:
        z = x @ W
        if b is not None:
            z = z + (b.to(z.dtype) if b.dtype != z.dtype else b)
    return activation(z, training) if activation is not None else z


def layer_norm(x, gain, bias=None, eps=1e-5, residual=None):
    """Layer norm over the last axis; with ``residual`` the input is ``x + residual`` (added inside the kernel)."""
    nat = _native_for(x)
    if nat is not None and x.dtype in (torch.bfloat16, torch.float16, torch.float32) and x.shape[-1] % 8 == 0:
        y = nat.layer_norm(x, gain, bias, eps, residual)
        if y is not None:
            return y
    if residual is not None:
        x = x + residual
    return F.layer_norm(x, (x.shape[-1],), gain.to(x.dtype), None if bias is None else bias.to(x.dtype), eps)


def softmax_xent(logits, labels, sparse=False):
    """Per-row softmax cross-entropy: ``labels`` one-hot/probabilities [N,C] or indices [N]."""
    nat = _native_for(logits)
    if nat is not None:
        y = nat.softmax_xent(logits, labels, sparse)
        if y is not None:
            return y
    lp = F.log_softmax(_up(logits), dim=-1)
    if sparse:
        return -lp.gather(1, labels.reshape(-1, 1).long()).reshape(-1)
    return -(labels.to(lp.dtype) * lp).sum(-1)


def gelu(x, approximate="none"):
    if approximate == "sigmoid":
        return x * torch.sigmoid(1.702 * x)
    return F.gelu(x, approximate=approximate)


def attention(q, k, v, mask=None, scale=None, dropout_p=0.0, training=False):
    """Scaled dot-product attention over [B, H, T, D] tensors; ``mask`` is [B, Tk] (1 = keep)."""
    nat = _native_for(q)
    if nat is not None and q.dtype in (torch.bfloat16, torch.float16):
        y = nat.attention(q, k, v, mask, scale, dropout_p if training else 0.0)      # dropout inside the fused kernels
        if y is not None:
            return y
    d = q.shape[-1]
    scale = scale if scale is not None else d ** -0.5
    s = torch.matmul(q, k.transpose(-1, -2)) * scale
    if mask is not None:
        s = s.masked_fill(mask[:, None, None, :] == 0, float("-inf")) if mask.dim() == 2 else s + mask
    p = torch.softmax(_up(s), dim=-1).to(q.dtype)
    if dropout_p > 0.0 and training:
        p = F.dropout(p, dropout_p, True)
    return torch.matmul(p, v)


def lstm_cell(z, c_prev, gate_act=torch.sigmoid, act=torch.tanh):
    """DL4J LSTM cell from pre-activations ``z`` [mb, 4n] in gate order [i(block input), f, o, g].

    Reference: ``nn/layers/recurrent/LSTMHelpers.java:180-330`` — block input ``a=act(z_i)``,
    forget ``f=σ(z_f)``, output ``o=σ(z_o)``, input-modulation ``g=σ(z_g)``;
    ``c = f*c_prev + g*a``; ``h = o*act(c)``.
    """
    nat = _native_for(z)
    if nat is not None and gate_act is torch.sigmoid and act is torch.tanh:
        r = nat.lstm_cell(z, c_prev)
        if r is not None:
            return r
    n = z.shape[1] // 4
    a = act(z[:, :n])
    f = gate_act(z[:, n:2 * n])
    o = gate_act(z[:, 2 * n:3 * n])
    g = gate_act(z[:, 3 * n:])
    c = f * c_prev + g * a
    h = o * act(c)
    return h, c
