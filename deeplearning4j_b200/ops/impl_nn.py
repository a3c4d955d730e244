"""NN ops (``headers/nn.h`` + nn-related parity ops): softmax family, layer/batch norm, lrn,
dropout, bias add, xw_plus_b / relu_layer, attention ops, matmul family.

The hot ones route through ``ops.nnops`` so that on a B200 they run on the hand-written kernels
(tcgen05 GEMM with fused epilogues, fused layer norm, batched-GEMM attention)."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import nnops
from .registry import op


def _ints(v):
    if v is None:
        return None
    if isinstance(v, torch.Tensor):
        return [int(e) for e in v.reshape(-1).tolist()]
    if isinstance(v, (int, float)):
        return [int(v)]
    return [int(e) for e in v]


def _autobp(fn, n_in):
    """Build a ``*_bp`` op from ``fn`` for its first ``n_in`` tensor inputs via autograd."""
    def run(*args, **kw):
        *xs, g = args
        xs = list(xs)
        leaves = [x.detach().requires_grad_(True) if i < n_in and x is not None and x.dtype.is_floating_point else x
                  for i, x in enumerate(xs)]
        with torch.enable_grad():
            y = fn(*leaves, **kw)
        diff = [l for i, l in enumerate(leaves) if i < n_in and l is not None and l.requires_grad]
        grads = torch.autograd.grad(y, diff, g.reshape(y.shape).to(y.dtype), allow_unused=True)
        grads = [gr if gr is not None else torch.zeros_like(l) for gr, l in zip(grads, diff)]
        return tuple(grads) if len(grads) > 1 else grads[0]
    return run


# ----------------------------------------------------------------------------- softmax family
@op("softmax")
def softmax(x, dimension=-1, **kw):
    return torch.softmax(x, dim=int(dimension))


@op("log_softmax")
def log_softmax(x, dimension=-1, **kw):
    return torch.log_softmax(x, dim=int(dimension))


op("softmax_bp")(_autobp(softmax, 1))
op("log_softmax_bp")(_autobp(log_softmax, 1))


# ----------------------------------------------------------------------------- matmul family
def _mm(a, b):
    if a.dim() == 2 and b.dim() == 2:
        from . import linalg_dispatch
        return linalg_dispatch.matmul(a, b)
    return torch.matmul(a, b)


@op("matmul", "mmul")
def matmul(x, y, transposeX=False, transposeY=False, transposeZ=False, alpha=1.0, beta=0.0, **kw):
    a = x.transpose(-1, -2) if transposeX and x.dim() > 1 else x
    b = y.transpose(-1, -2) if transposeY and y.dim() > 1 else y
    z = _mm(a, b)
    if alpha != 1.0:
        z = z * alpha
    return z.transpose(-1, -2) if transposeZ and z.dim() > 1 else z


op("matmul_bp", n_out=2)(_autobp(matmul, 2))


@op("tensormmul")
def tensormmul(x, y, axes_x=None, axes_y=None, dimensionsX=None, dimensionsY=None, **kw):
    ax = _ints(dimensionsX if dimensionsX is not None else axes_x)
    ay = _ints(dimensionsY if dimensionsY is not None else axes_y)
    return torch.tensordot(x, y, dims=(ax, ay))


op("tensormmul_bp", n_out=2)(_autobp(tensormmul, 2))


@op("batched_gemm", n_out=-1)
def batched_gemm(*args, transposeA=False, transposeB=False, M=None, N=None, K=None, batchSize=None, **kw):
    # native layout: alpha, beta, A_0..A_{b-1}, B_0..B_{b-1}
    alpha, beta, rest = args[0], args[1], args[2:]
    nb = len(rest) // 2
    outs = []
    for i in range(nb):
        a = rest[i].t() if transposeA else rest[i]
        b = rest[nb + i].t() if transposeB else rest[nb + i]
        outs.append(_mm(a, b) * alpha.reshape(-1)[min(i, alpha.numel() - 1)])
    return tuple(outs)


@op("batched_gemm_bp", n_out=-1)
def batched_gemm_bp(*args, transposeA=False, transposeB=False, **kw):
    # inputs: alpha, beta, A_0.., B_0.., dC_0..  ->  dA_0.., dB_0..
    alpha, beta, rest = args[0], args[1], args[2:]
    nb = len(rest) // 3
    A, B, dC = rest[:nb], rest[nb:2 * nb], rest[2 * nb:]
    dA, dB = [], []
    for a, b, g in zip(A, B, dC):
        al = alpha.reshape(-1)[0]
        aa = a.t() if transposeA else a
        bb = b.t() if transposeB else b
        ga, gb = (g @ bb.t()) * al, (aa.t() @ g) * al
        dA.append(ga.t() if transposeA else ga)
        dB.append(gb.t() if transposeB else gb)
    return tuple(dA) + tuple(dB)


@op("xw_plus_b", "linear")
def xw_plus_b(x, w, b=None, transposeW=False, aTranspose=False, **kw):
    W = w.t() if transposeW else w
    if x.dim() == 2:
        return nnops.linear(x, W, b)
    lead = x.shape[:-1]
    return nnops.linear(x.reshape(-1, x.shape[-1]), W, b).reshape(*lead, W.shape[1])


op("xw_plus_b_bp", n_out=3)(_autobp(xw_plus_b, 3))


@op("relu_layer")
def relu_layer(x, w, b, **kw):
    from ..nn.activations import ActivationReLU
    return nnops.linear(x, w, b, ActivationReLU())


@op("linear_gelu")
def linear_gelu(x, w, b=None, precise=False, **kw):
    """Fused ``gelu(x @ w + b)``: produced by the graph optimizer from ``xw_plus_b`` -> ``gelu``."""
    from ..nn.activations import ActivationGELU
    if x.dim() == 2:
        return nnops.linear(x, w, b, ActivationGELU(precise))
    lead = x.shape[:-1]
    return nnops.linear(x.reshape(-1, x.shape[-1]), w, b, ActivationGELU(precise)).reshape(*lead, w.shape[1])


@op("mlp_gelu")
def mlp_gelu(x, w1, b1, w2, b2=None, precise=False, **kw):
    """Fused ``gelu(x @ w1 + b1) @ w2 + b2``: produced by the graph optimizer from ``xw_plus_b -> gelu -> xw_plus_b``; on the native
    path the GELU gradient is applied inside the second layer's data-gradient GEMM."""
    from ..nn.activations import ActivationGELU
    act = ActivationGELU(precise)
    lead = x.shape[:-1]
    x2 = x if x.dim() == 2 else x.reshape(-1, x.shape[-1])
    nat = nnops._native_for(x2)
    y = nat.mlp(x2, w1, b1, w2, b2, act) if nat is not None and x2.dtype in (torch.bfloat16, torch.float16) else None
    if y is None:
        y = nnops.linear(nnops.linear(x2, w1, b1, act), w2, b2, None)
    return y if x.dim() == 2 else y.reshape(*lead, w2.shape[1])


@op("biasadd")
def biasadd(x, b, nchw=False, **kw):
    if nchw and x.dim() > 2:
        return x + b.reshape([1, -1] + [1] * (x.dim() - 2))
    return x + b


@op("biasadd_bp", n_out=2)
def biasadd_bp(x, b, g, nchw=False, **kw):
    dims = [i for i in range(x.dim()) if i != (1 if nchw and x.dim() > 2 else x.dim() - 1)]
    return g, g.sum(dims)


# ----------------------------------------------------------------------------- normalisation
@op("layer_norm")
def layer_norm(x, gain, bias=None, dimensions=(-1,), channelsFirst=False, **kw):
    dims = _ints(dimensions) or [-1]
    dims = [d % x.dim() for d in dims]
    if dims == [x.dim() - 1]:
        # a 1-D parameter is passed as is: reshape would return a view without the link to its fp32 master
        flat = lambda t: t if t is None or t.dim() == 1 else t.reshape(-1)
        return nnops.layer_norm(x, flat(gain), flat(bias), 1e-5)
    mean = x.mean(dims, keepdim=True)
    var = x.var(dims, unbiased=False, keepdim=True)
    shape = [x.shape[d] if d in dims else 1 for d in range(x.dim())]
    y = (x - mean) / torch.sqrt(var + 1e-5) * gain.reshape(shape)
    return y + bias.reshape(shape) if bias is not None else y


op("layer_norm_bp", n_out=3)(_autobp(layer_norm, 3))


@op("add_layer_norm")
def add_layer_norm(a, b, gain, bias=None, dimensions=(-1,), channelsFirst=False, **kw):
    """Fused ``layer_norm(a + b)``: produced by the session from ``add`` -> ``layer_norm`` (the residual connections of a
    transformer block); falls back to the two ops when the operands broadcast or the axis is not the last one."""
    dims = [d % a.dim() for d in (_ints(dimensions) or [-1])]
    if a.shape == b.shape and a.dtype == b.dtype and dims == [a.dim() - 1]:
        flat = lambda t: t if t is None or t.dim() == 1 else t.reshape(-1)
        return nnops.layer_norm(a, flat(gain), flat(bias), 1e-5, residual=b)
    return layer_norm(a + b, gain, bias, dimensions=dimensions, channelsFirst=channelsFirst)


@op("standardize")
def standardize(x, dimensions=(-1,), **kw):
    d = [i % x.dim() for i in (_ints(dimensions) or [-1])]
    return (x - x.mean(d, keepdim=True)) / x.std(d, unbiased=False, keepdim=True).clamp_min(1e-12)


op("standardize_bp")(_autobp(standardize, 1))


@op("batchnorm")
def batchnorm(x, mean, variance, gamma=None, beta=None, epsilon=1e-5, applyScale=None, applyOffset=None, axis=(1,), **kw):
    ax = [a % x.dim() for a in (_ints(axis) or [1])]
    shape = [x.shape[d] if d in ax else 1 for d in range(x.dim())]
    y = (x - mean.reshape(shape)) / torch.sqrt(variance.reshape(shape) + epsilon)
    if gamma is not None and applyScale is not False:
        y = y * gamma.reshape(shape)
    if beta is not None and applyOffset is not False:
        y = y + beta.reshape(shape)
    return y


op("batchnorm_bp", n_out=-1)(_autobp(batchnorm, 5))


@op("fused_batch_norm", n_out=3)
def fused_batch_norm(x, scale, offset, mean=None, variance=None, epsilon=1e-3, dataFormat=0, isTraining=True, **kw):
    nchw = bool(dataFormat)
    xc = x if nchw else x.permute(0, 3, 1, 2)
    if isTraining or mean is None or mean.numel() == 0:
        m = xc.mean((0, 2, 3))
        v = xc.var((0, 2, 3), unbiased=False)
    else:
        m, v = mean, variance
    y = F.batch_norm(xc, m, v, scale, offset, False, 0.0, epsilon)
    return (y if nchw else y.permute(0, 2, 3, 1)), m, v


@op("lrn")
def lrn(x, depth=5, bias=1.0, alpha=1.0, beta=0.5, **kw):
    n = 2 * int(depth) + 1
    return F.local_response_norm(x, n, alpha=alpha * n, beta=beta, k=bias)


op("lrn_bp")(_autobp(lrn, 1))


@op("dropout")
def dropout(x, probValue=0.5, seed=None, inverted=True, training=True, **kw):
    """``probValue`` is the retain probability (DL4J / libnd4j convention)."""
    if not training or probValue >= 1.0:
        return x
    return F.dropout(x, 1.0 - float(probValue), True)


op("dropout_bp")(lambda x, g, probValue=0.5, **kw: g)
op("alpha_dropout_bp")(lambda x, g, **kw: g)
op("dropout_inverted")(dropout)


@op("apply_sgd")
def apply_sgd(params, grads, lr=None, learningRate=0.01, **kw):
    l = float(lr) if lr is not None else learningRate
    return params - l * grads


# ----------------------------------------------------------------------------- attention
@op("dot_product_attention", n_out=-1)
def dot_product_attention(q, k, v, mask=None, scaled=True, withWeights=False, **kw):
    """q [B, d, Tq] / k [B, d, Tk] / v [B, dv, Tk] (or 4-D with a heads axis after batch), features-first
    as in the native op (``generic/nn/dot_product_attention.cpp``)."""
    four = q.dim() == 4
    qq = (q if four else q.unsqueeze(1)).transpose(-1, -2)
    kk = (k if four else k.unsqueeze(1)).transpose(-1, -2)
    vv = (v if four else v.unsqueeze(1)).transpose(-1, -2)
    scale = (1.0 / math.sqrt(q.shape[-2])) if scaled else 1.0
    if withWeights:
        s = torch.matmul(qq, kk.transpose(-1, -2)) * scale
        if mask is not None:
            s = s.masked_fill(mask.reshape(mask.shape[0], 1, 1, -1) == 0, float("-inf"))
        w = torch.softmax(s.float(), -1).to(q.dtype)
        o = torch.matmul(w, vv).transpose(-1, -2)
        return (o if four else o.squeeze(1)), (w.transpose(-1, -2) if four else w.squeeze(1).transpose(-1, -2))
    o = nnops.attention(qq, kk, vv, mask, scale).transpose(-1, -2)
    return (o if four else o.squeeze(1),)


@op("dot_product_attention_v2", n_out=-1)
def dot_product_attention_v2(q, v, k=None, attentionBias=None, qMask=None, vMask=None, scale=1.0, dropoutProbability=0.0,
                             useCausalMask=False, training=False, **kw):
    """Batch-major variant: q [B, (H,) Tq, d], v/k [B, (H,) Tk, d]."""
    k = v if k is None else k
    four = q.dim() == 4
    qq, kk, vv = (t if four else t.unsqueeze(1) for t in (q, k, v))
    sc = float(scale) if scale else 1.0
    mask = vMask
    if useCausalMask or attentionBias is not None or qMask is not None:
        s = torch.matmul(qq, kk.transpose(-1, -2)) * sc
        if attentionBias is not None:
            s = s + attentionBias
        if useCausalMask:
            T1, T2 = s.shape[-2:]
            s = s.masked_fill(torch.ones(T1, T2, dtype=torch.bool, device=s.device).triu(1), float("-inf"))
        if vMask is not None:
            s = s.masked_fill(vMask.reshape(vMask.shape[0], 1, 1, -1) == 0, float("-inf"))
        w = torch.softmax(s.float(), -1).to(q.dtype)
        if dropoutProbability and training:
            w = F.dropout(w, dropoutProbability, True)
        o = torch.matmul(w, vv)
        if qMask is not None:
            o = o * qMask.reshape(qMask.shape[0], 1, -1, 1).to(o.dtype)
    else:
        o = nnops.attention(qq, kk, vv, mask, sc, dropoutProbability, training)
    return (o if four else o.squeeze(1),)


@op("multi_head_dot_product_attention", n_out=-1)
def multi_head_dot_product_attention(q, k, v, Wq, Wk, Wv, Wo, mask=None, scaled=True, withWeights=False, **kw):
    """q/k/v [B, nIn, T] features-first; Wq/Wk/Wv [H, dh, nIn]; Wo [H*dh, nOut] -> [B, nOut, Tq]
    (``generic/nn/multi_head_dot_product_attention.cpp:99-134``).  When q, k and v are the same tensor
    the three projections are one GEMM over the concatenated weights."""
    B, nIn, Tq = q.shape
    H, dh = Wq.shape[0], Wq.shape[1]

    def rows(x):
        return x.permute(0, 2, 1).reshape(-1, x.shape[1])
    if q is k and k is v:
        Wcat = torch.cat([Wq.reshape(H * dh, nIn), Wk.reshape(H * dh, nIn), Wv.reshape(H * dh, nIn)], 0).t()
        qkv = nnops.linear(rows(q), Wcat.to(q.dtype), None).reshape(B, Tq, 3, H, dh)
        qq, kk, vv = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    else:
        def proj(x, W):
            y = nnops.linear(rows(x), W.reshape(H * dh, -1).t().to(x.dtype), None)
            return y.reshape(x.shape[0], x.shape[2], H, dh).permute(0, 2, 1, 3)
        qq, kk, vv = proj(q, Wq), proj(k, Wk), proj(v, Wv)
    scale = 1.0 / math.sqrt(dh) if scaled else 1.0
    o = nnops.attention(qq, kk, vv, mask, scale)                     # [B, H, Tq, dh]
    o = o.permute(0, 2, 1, 3).reshape(B * Tq, H * dh)
    y = nnops.linear(o, Wo.to(o.dtype), None).reshape(B, Tq, -1).permute(0, 2, 1)
    return (y,)


op("dot_product_attention_bp", n_out=3)(_autobp(lambda q, k, v, **kw: dot_product_attention(q, k, v, **kw)[0], 3))
op("dot_product_attention_v2_bp", n_out=3)(_autobp(lambda q, v, k, **kw: dot_product_attention_v2(q, v, k, **kw)[0], 3))
op("multi_head_dot_product_attention_bp", n_out=7)(
    _autobp(lambda q, k, v, a, b, c, d, **kw: multi_head_dot_product_attention(q, k, v, a, b, c, d, **kw)[0], 7))


# ----------------------------------------------------------------------------- clipping
@op("clipbynorm")
def clipbynorm(x, clipValue=1.0, dimensions=None, **kw):
    d = _ints(dimensions)
    n = torch.linalg.vector_norm(x, dim=d, keepdim=True) if d else torch.linalg.vector_norm(x)
    return torch.where(n > clipValue, x * (clipValue / n.clamp_min(1e-30)), x)


op("clipbynorm_bp")(_autobp(clipbynorm, 1))


@op("clipbyavgnorm")
def clipbyavgnorm(x, clipValue=1.0, dimensions=None, **kw):
    d = _ints(dimensions)
    cnt = x.numel() if not d else math.prod(x.shape[i] for i in d)
    n = (torch.linalg.vector_norm(x, dim=d, keepdim=True) if d else torch.linalg.vector_norm(x)) / cnt
    return torch.where(n > clipValue, x * (clipValue / n.clamp_min(1e-30)), x)


op("clipbyavgnorm_bp")(_autobp(clipbyavgnorm, 1))


@op("clip_by_global_norm", n_out=-1)
def clip_by_global_norm(*xs, clipNorm=1.0, **kw):
    g = torch.sqrt(sum((x.float() ** 2).sum() for x in xs))
    s = clipNorm / torch.maximum(g, torch.tensor(clipNorm, device=g.device))
    return tuple(x * s.to(x.dtype) for x in xs) + (g,)


# ----------------------------------------------------------------------------- merge ops
op("mergeadd", "mergesum")(lambda *xs, **kw: torch.stack(xs).sum(0))
op("mergeavg")(lambda *xs, **kw: torch.stack(xs).mean(0))
op("mergemax")(lambda *xs, **kw: torch.stack(xs).amax(0))
op("mergemaxindex", differentiable=False)(lambda *xs, **kw: torch.stack(xs).argmax(0))
op("mergeadd_bp", n_out=-1)(lambda *a, **kw: tuple(a[-1] for _ in a[:-1]))
op("mergeavg_bp", n_out=-1)(lambda *a, **kw: tuple(a[-1] / (len(a) - 1) for _ in a[:-1]))


@op("mergemax_bp", n_out=-1)
def mergemax_bp(*a, **kw):
    xs, g = a[:-1], a[-1]
    idx = torch.stack(xs).argmax(0)
    return tuple(g * (idx == i).to(g.dtype) for i in range(len(xs)))
