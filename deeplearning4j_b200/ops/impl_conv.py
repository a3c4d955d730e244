"""Convolution / pooling ops (``headers/convo.h``): conv1d/2d/3d, depthwise, separable, pointwise,
deconv, pooling 2d/3d, upsampling, im2col/col2im, dilation2d, ismax.  Argument names follow the
Conv*Config objects of the Java API (kH, kW, sH, sW, pH, pW, dH, dW, isSameMode/paddingMode,
dataFormat: 0 = NCHW, 1 = NHWC; weights format 0 = [kH,kW,iC,oC] (YXIO), 1 = [oC,iC,kH,kW], 2 = [oC,kH,kW,iC];
``libnd4j/include/ops/declarable/helpers/cuda/convolutions_conv2d.cu:36-39``)."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .registry import op
from .impl_nn import _autobp


def _same_pad(size, k, s, d):
    out = -(-size // s)
    total = max((out - 1) * s + (k - 1) * d + 1 - size, 0)
    return total // 2, total - total // 2


def _prep(x, ks, ss, ps, ds, same, value=0.0):
    if not same:
        return x, list(ps)
    pads = [_same_pad(x.shape[2 + i], ks[i], ss[i], ds[i]) for i in range(len(ks))]
    if all(lo == hi for lo, hi in pads):
        return x, [p[0] for p in pads]
    flat = []
    for lo, hi in reversed(pads):
        flat += [lo, hi]
    return F.pad(x, flat, value=value), [0] * len(ks)


def _w2d(w, wFormat):
    wFormat = int(wFormat)
    if wFormat == 0:
        return w.permute(3, 2, 0, 1)
    if wFormat == 2:
        return w.permute(0, 3, 1, 2)
    return w


def _is_same(isSameMode, paddingMode):
    if paddingMode is not None:
        return str(paddingMode).upper() in ("SAME", "1") or paddingMode == 1
    return bool(isSameMode)


@op("conv2d")
def conv2d(x, w, b=None, kH=None, kW=None, sH=1, sW=1, pH=0, pW=0, dH=1, dW=1, isSameMode=False, paddingMode=None,
           dataFormat=0, wFormat=0, isNHWC=None, **kw):
    nhwc = bool(dataFormat) if isNHWC is None else bool(isNHWC)
    xc = x.permute(0, 3, 1, 2) if nhwc else x
    W = _w2d(w, wFormat)
    xc, pad = _prep(xc, W.shape[2:], (sH, sW), (pH, pW), (dH, dW), _is_same(isSameMode, paddingMode))
    y = F.conv2d(xc, W.to(xc.dtype), None if b is None else b.reshape(-1).to(xc.dtype), (sH, sW), tuple(pad), (dH, dW))
    return y.permute(0, 2, 3, 1) if nhwc else y


op("conv2d_bp", n_out=-1)(_autobp(conv2d, 3))
op("conv2d_input_bp")(lambda shape, w, g, **kw: _autobp(conv2d, 1)(torch.zeros([int(s) for s in shape.tolist()], dtype=g.dtype, device=g.device), w, g, **kw))
op("pointwise_conv2d")(lambda x, w, b=None, dataFormat=0, wFormat=0, **kw: conv2d(x, w, b, dataFormat=dataFormat, wFormat=wFormat))


@op("conv1d")
def conv1d(x, w, b=None, k=None, s=1, p=0, d=1, isSameMode=False, paddingMode=None, dataFormat=0, wFormat=0, isNWC=None, **kw):
    nwc = bool(dataFormat) if isNWC is None else bool(isNWC)
    xc = x.permute(0, 2, 1) if nwc else x
    wf = int(wFormat)
    W = w.permute(2, 1, 0) if wf == 0 else (w.permute(0, 2, 1) if wf == 2 else w)     # -> [oC, iC, k]
    pm = str(paddingMode).upper() if paddingMode is not None else None
    if pm in ("CAUSAL", "2"):
        xc, pad = F.pad(xc, [(W.shape[2] - 1) * d, 0]), [0]
    else:
        xc, pad = _prep(xc, W.shape[2:], (s,), (p,), (d,), _is_same(isSameMode, paddingMode))
    y = F.conv1d(xc, W.to(xc.dtype), None if b is None else b.reshape(-1).to(xc.dtype), s, pad[0], d)
    return y.permute(0, 2, 1) if nwc else y


op("conv1d_bp", n_out=-1)(_autobp(conv1d, 3))


@op("conv3dnew", "conv3d")
def conv3dnew(x, w, b=None, kD=None, kH=None, kW=None, sD=1, sH=1, sW=1, pD=0, pH=0, pW=0, dD=1, dH=1, dW=1,
              isSameMode=False, paddingMode=None, dataFormat=0, wFormat=0, isNCDHW=None, **kw):
    ncdhw = (not bool(dataFormat)) if isNCDHW is None else bool(isNCDHW)
    xc = x if ncdhw else x.permute(0, 4, 1, 2, 3)
    wf = int(wFormat)
    W = w.permute(4, 3, 0, 1, 2) if wf == 0 else (w.permute(0, 4, 1, 2, 3) if wf == 2 else w)
    xc, pad = _prep(xc, W.shape[2:], (sD, sH, sW), (pD, pH, pW), (dD, dH, dW), _is_same(isSameMode, paddingMode))
    y = F.conv3d(xc, W.to(xc.dtype), None if b is None else b.reshape(-1).to(xc.dtype), (sD, sH, sW), tuple(pad), (dD, dH, dW))
    return y if ncdhw else y.permute(0, 2, 3, 4, 1)


op("conv3dnew_bp", n_out=-1)(_autobp(conv3dnew, 3))


@op("depthwise_conv2d")
def depthwise_conv2d(x, w, b=None, sH=1, sW=1, pH=0, pW=0, dH=1, dW=1, isSameMode=False, paddingMode=None, dataFormat=0,
                     wFormat=0, **kw):
    nhwc = bool(dataFormat)
    xc = x.permute(0, 3, 1, 2) if nhwc else x
    wf = int(wFormat)
    Wk = w if wf == 0 else (w.permute(2, 3, 1, 0) if wf == 1 else w.permute(1, 2, 3, 0))   # -> [kH,kW,iC,mC]
    kH, kW, iC, mC = Wk.shape
    W = Wk.permute(2, 3, 0, 1).reshape(iC * mC, 1, kH, kW)
    xc, pad = _prep(xc, (kH, kW), (sH, sW), (pH, pW), (dH, dW), _is_same(isSameMode, paddingMode))
    y = F.conv2d(xc, W.to(xc.dtype), None if b is None else b.reshape(-1).to(xc.dtype), (sH, sW), tuple(pad), (dH, dW), groups=iC)
    return y.permute(0, 2, 3, 1) if nhwc else y


op("depthwise_conv2d_bp", n_out=-1)(_autobp(depthwise_conv2d, 3))


@op("sconv2d")
def sconv2d(x, wd, wp=None, b=None, sH=1, sW=1, pH=0, pW=0, dH=1, dW=1, isSameMode=False, paddingMode=None, dataFormat=0,
            wFormat=0, **kw):
    y = depthwise_conv2d(x, wd, None if wp is not None else b, sH, sW, pH, pW, dH, dW, isSameMode, paddingMode, dataFormat, wFormat)
    if wp is not None:
        y = conv2d(y, wp, b, dataFormat=dataFormat, wFormat=wFormat)
    return y


op("sconv2d_bp", n_out=-1)(_autobp(sconv2d, 4))


@op("deconv2d", "deconv2d_tf")
def deconv2d(x, w, b=None, sH=1, sW=1, pH=0, pW=0, dH=1, dW=1, isSameMode=False, paddingMode=None, dataFormat=0, wFormat=0, **kw):
    nhwc = bool(dataFormat)
    xc = x.permute(0, 3, 1, 2) if nhwc else x
    wf = int(wFormat)
    W = w.permute(3, 2, 0, 1) if wf == 0 else (w.permute(3, 0, 1, 2) if wf == 2 else w.permute(1, 0, 2, 3))   # -> [iC, oC, kH, kW]
    same = _is_same(isSameMode, paddingMode)
    y = F.conv_transpose2d(xc, W.to(xc.dtype), None if b is None else b.reshape(-1).to(xc.dtype), (sH, sW),
                           (0, 0) if same else (pH, pW), dilation=(dH, dW))
    if same:
        th, tw = xc.shape[2] * sH, xc.shape[3] * sW
        oh, ow = (y.shape[2] - th) // 2, (y.shape[3] - tw) // 2
        y = y[:, :, oh:oh + th, ow:ow + tw]
    return y.permute(0, 2, 3, 1) if nhwc else y


op("deconv2d_bp", n_out=-1)(_autobp(deconv2d, 3))


@op("deconv3d")
def deconv3d(x, w, b=None, sD=1, sH=1, sW=1, pD=0, pH=0, pW=0, dD=1, dH=1, dW=1, isSameMode=False, paddingMode=None,
             dataFormat=0, wFormat=0, **kw):
    ncdhw = not bool(dataFormat)
    xc = x if ncdhw else x.permute(0, 4, 1, 2, 3)
    wf = int(wFormat)
    W = w.permute(4, 3, 0, 1, 2) if wf == 0 else w.permute(1, 0, 2, 3, 4)
    same = _is_same(isSameMode, paddingMode)
    y = F.conv_transpose3d(xc, W.to(xc.dtype), None if b is None else b.reshape(-1).to(xc.dtype), (sD, sH, sW),
                           (0, 0, 0) if same else (pD, pH, pW), dilation=(dD, dH, dW))
    if same:
        tgt = [xc.shape[2] * sD, xc.shape[3] * sH, xc.shape[4] * sW]
        off = [(y.shape[2 + i] - tgt[i]) // 2 for i in range(3)]
        y = y[:, :, off[0]:off[0] + tgt[0], off[1]:off[1] + tgt[1], off[2]:off[2] + tgt[2]]
    return y if ncdhw else y.permute(0, 2, 3, 4, 1)


op("deconv3d_bp", n_out=-1)(_autobp(deconv3d, 3))


# ----------------------------------------------------------------------------- pooling
def _pool2d(kind):
    def run(x, kH=2, kW=2, sH=2, sW=2, pH=0, pW=0, dH=1, dW=1, isSameMode=False, paddingMode=None, extraParam0=0, dataFormat=0,
            isNHWC=None, pnorm=2, **kw):
        nhwc = bool(dataFormat) if isNHWC is None else bool(isNHWC)
        xc = x.permute(0, 3, 1, 2) if nhwc else x
        fill = float("-inf") if kind == "max" else 0.0
        xc, pad = _prep(xc, (kH, kW), (sH, sW), (pH, pW), (dH, dW), _is_same(isSameMode, paddingMode), fill)
        if kind == "max":
            y = F.max_pool2d(xc, (kH, kW), (sH, sW), tuple(pad), (dH, dW))
        elif kind == "avg":
            y = F.avg_pool2d(xc, (kH, kW), (sH, sW), tuple(pad), count_include_pad=bool(extraParam0) or True)
        else:
            p = float(extraParam0 or pnorm)
            y = (F.avg_pool2d(xc.abs() ** p, (kH, kW), (sH, sW), tuple(pad)) * (kH * kW)) ** (1.0 / p)
        return y.permute(0, 2, 3, 1) if nhwc else y
    return run


for _k, _n in (("max", "maxpool2d"), ("avg", "avgpool2d"), ("pnorm", "pnormpool2d")):
    _f = _pool2d(_k)
    op(_n)(_f)
    op(_n + "_bp")(_autobp(_f, 1))


def _pool3d(kind):
    def run(x, kD=2, kH=2, kW=2, sD=2, sH=2, sW=2, pD=0, pH=0, pW=0, dD=1, dH=1, dW=1, isSameMode=False, paddingMode=None,
            extraParam0=0, dataFormat=0, isNCDHW=None, **kw):
        ncdhw = (not bool(dataFormat)) if isNCDHW is None else bool(isNCDHW)
        xc = x if ncdhw else x.permute(0, 4, 1, 2, 3)
        fill = float("-inf") if kind == "max" else 0.0
        xc, pad = _prep(xc, (kD, kH, kW), (sD, sH, sW), (pD, pH, pW), (dD, dH, dW), _is_same(isSameMode, paddingMode), fill)
        if kind == "max":
            y = F.max_pool3d(xc, (kD, kH, kW), (sD, sH, sW), tuple(pad), (dD, dH, dW))
        else:
            y = F.avg_pool3d(xc, (kD, kH, kW), (sD, sH, sW), tuple(pad))
        return y if ncdhw else y.permute(0, 2, 3, 4, 1)
    return run


for _k, _n in (("max", "maxpool3dnew"), ("avg", "avgpool3dnew")):
    _f = _pool3d(_k)
    op(_n)(_f)
    op(_n + "_bp")(_autobp(_f, 1))


@op("max_pool_with_argmax", n_out=2)
def max_pool_with_argmax(x, kH=2, kW=2, sH=2, sW=2, pH=0, pW=0, dH=1, dW=1, isSameMode=False, dataFormat=1, **kw):
    nhwc = bool(dataFormat)
    xc = x.permute(0, 3, 1, 2) if nhwc else x
    xc, pad = _prep(xc, (kH, kW), (sH, sW), (pH, pW), (dH, dW), bool(isSameMode), float("-inf"))
    y, idx = F.max_pool2d(xc, (kH, kW), (sH, sW), tuple(pad), (dH, dW), return_indices=True)
    # flattened position inside one example as the reference (and TensorFlow) count it: ((row * W) + column) * C + channel
    C = xc.shape[1]
    idx = idx * C + torch.arange(C, device=idx.device).reshape(1, C, 1, 1)
    return (y.permute(0, 2, 3, 1), idx.permute(0, 2, 3, 1)) if nhwc else (y, idx)


@op("upsampling2d")
def upsampling2d(x, scaleH=2, scaleW=2, nchw=True, **kw):
    d = (2, 3) if nchw else (1, 2)
    return x.repeat_interleave(int(scaleH), d[0]).repeat_interleave(int(scaleW), d[1])


op("upsampling2d_bp")(_autobp(upsampling2d, 1))


@op("upsampling3d")
def upsampling3d(x, scaleD=2, scaleH=2, scaleW=2, ncdhw=True, **kw):
    d = (2, 3, 4) if ncdhw else (1, 2, 3)
    return x.repeat_interleave(int(scaleD), d[0]).repeat_interleave(int(scaleH), d[1]).repeat_interleave(int(scaleW), d[2])


op("upsampling3d_bp")(_autobp(upsampling3d, 1))


@op("im2col")
def im2col(x, kH=2, kW=2, sH=1, sW=1, pH=0, pW=0, dH=1, dW=1, isSameMode=False, zeroPadVal=0.0, **kw):
    xc, pad = _prep(x, (kH, kW), (sH, sW), (pH, pW), (dH, dW), bool(isSameMode), zeroPadVal)
    n, c = xc.shape[:2]
    cols = F.unfold(xc, (kH, kW), (dH, dW), tuple(pad), (sH, sW))
    oh = (xc.shape[2] + 2 * pad[0] - (kH - 1) * dH - 1) // sH + 1
    ow = (xc.shape[3] + 2 * pad[1] - (kW - 1) * dW - 1) // sW + 1
    return cols.reshape(n, c, kH, kW, oh, ow)


op("im2col_bp")(_autobp(im2col, 1))


@op("col2im")
def col2im(cols, sH=1, sW=1, pH=0, pW=0, imgH=None, imgW=None, dH=1, dW=1, **kw):
    n, c, kH, kW, oh, ow = cols.shape
    return F.fold(cols.reshape(n, c * kH * kW, oh * ow), (int(imgH), int(imgW)), (kH, kW), (dH, dW), (pH, pW), (sH, sW))


@op("dilation2d")
def dilation2d(x, w, sH=1, sW=1, rH=1, rW=1, isSameMode=False, **kw):
    # NHWC input, w [kH, kW, C]: out = max_{ij}(x[h*s+i*r, w*s+j*r, c] + w[i,j,c])
    xc = x.permute(0, 3, 1, 2)
    kH, kW, C = w.shape
    xc, pad = _prep(xc, (kH, kW), (sH, sW), (0, 0), (rH, rW), bool(isSameMode), float("-inf"))
    n = xc.shape[0]
    cols = F.unfold(xc, (kH, kW), (rH, rW), tuple(pad), (sH, sW)).reshape(n, C, kH * kW, -1)
    y = (cols + w.permute(2, 0, 1).reshape(1, C, kH * kW, 1)).amax(2)
    oh = (xc.shape[2] + 2 * pad[0] - (kH - 1) * rH - 1) // sH + 1
    return y.reshape(n, C, oh, -1).permute(0, 2, 3, 1)


@op("ismax", differentiable=False)
def ismax(x, dimensions=None, **kw):
    if not dimensions:
        out = torch.zeros_like(x).reshape(-1)
        out[x.reshape(-1).argmax()] = 1
        return out.reshape(x.shape)
    d = int(dimensions[0] if isinstance(dimensions, (list, tuple)) else dimensions)
    return torch.zeros_like(x).scatter_(d, x.argmax(d, keepdim=True), 1.0)
