"""Convolution, pooling, padding, up-sampling and normalisation layers.

Parameter order/layout follows the reference initialisers: convolution ``b, W('c',[nOut,nIn,kH,kW])``
(``nn/params/ConvolutionParamInitializer.java:120-164``), depthwise ``b, W[kH,kW,nIn,mult]``,
separable ``b, dW, pW`` (``SeparableConvolutionParamInitializer.java``), batch-norm
``gamma, beta, mean, var|log10std`` (``BatchNormalizationParamInitializer.java:105-121``).
Activations use DL4J's logical NCHW axis order; on CUDA the tensors are kept in channels-last
memory format so that 1x1 convolutions are plain row-major GEMMs for the tcgen05 kernel.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ...ops import nnops
from ..conf.base import (BaseLayer, CNN2DFormat, ConvolutionMode, FeedForwardLayer, InputType, Layer, NoParamLayer,
                         ParamSpec, PoolingType, RNNFormat, _L)


def _pair(v, n=2):
    if v is None:
        return None
    if isinstance(v, (int, float)):
        return [int(v)] * n
    v = [int(e) for e in v]
    return v * n if len(v) == 1 else v


def conv_out_size(size, k, s, p, d, mode):
    eff = (k - 1) * d + 1
    if mode == ConvolutionMode.Same:
        return int(math.ceil(size / s))
    if mode == ConvolutionMode.Causal:
        return int(math.ceil(size / s))
    if mode == ConvolutionMode.Strict and (size - eff + 2 * p) % s != 0:
        raise ValueError(f"ConvolutionMode.Strict: (in={size} - k={eff} + 2*p={p}) not divisible by stride {s}")
    return (size - eff + 2 * p) // s + 1


def same_padding(size, k, s, d):
    out = int(math.ceil(size / s))
    total = max((out - 1) * s + (k - 1) * d + 1 - size, 0)
    return total // 2, total - total // 2


def _pad_for_mode(x, kernel, stride, padding, dilation, mode, value=0.0):
    """Returns (x possibly padded, symmetric padding list to hand to the torch op)."""
    nd = len(kernel)
    if mode == ConvolutionMode.Same:
        pads, sym = [], True
        for i in range(nd):
            lo, hi = same_padding(x.shape[2 + i], kernel[i], stride[i], dilation[i])
            pads.append((lo, hi))
            sym &= lo == hi
        if sym:
            return x, [p[0] for p in pads]
        flat = []
        for lo, hi in reversed(pads):
            flat += [lo, hi]
        return F.pad(x, flat, value=value), [0] * nd
    if mode == ConvolutionMode.Causal:
        lo = (kernel[0] - 1) * dilation[0]
        return F.pad(x, [lo, 0], value=value), [0] * nd
    return x, list(padding)


class ConvolutionLayer(FeedForwardLayer):
    JAVA_CLASS = _L + "ConvolutionLayer"
    DEFAULTS = {"hasBias": True, "convolutionMode": None, "dilation": [1, 1], "kernelSize": [5, 5], "stride": [1, 1],
                "padding": [0, 0], "cudnnAllowFallback": True, "cnn2dDataFormat": CNN2DFormat.NCHW,
                "cudnnAlgoMode": "PREFER_FASTEST", "cudnnFwdAlgo": None, "cudnnBwdFilterAlgo": None,
                "cudnnBwdDataAlgo": None}
    INHERIT = ("convolutionMode",)
    ND = 2

    def _positional(self, *args):
        names = ("kernelSize", "stride", "padding")
        for n, a in zip(names, args):
            setattr(self, n, a)
            self._explicit.add(n)

    def _finalise(self):
        super()._finalise()
        for f in ("kernelSize", "stride", "padding", "dilation"):
            setattr(self, f, _pair(getattr(self, f), self.ND))

    def _mode(self):
        return self.convolutionMode or ConvolutionMode.Truncate

    def setNIn(self, it, override):
        if self.nIn and not override:
            return
        self.nIn = it.channels if it.kind in (InputType.CNN, InputType.CNNFlat, InputType.CNN3D) else it.size

    def preprocessor_for(self, it):
        from ..conf.preprocessors import FeedForwardToCnnPreProcessor
        if it.kind == InputType.CNNFlat:
            return FeedForwardToCnnPreProcessor(it.height, it.width, it.channels)
        return None

    def output_type(self, it):
        h = conv_out_size(it.height, self.kernelSize[0], self.stride[0], self.padding[0], self.dilation[0], self._mode())
        w = conv_out_size(it.width, self.kernelSize[1], self.stride[1], self.padding[1], self.dilation[1], self._mode())
        return InputType.convolutional(h, w, self.nOut, getattr(it, "format", CNN2DFormat.NCHW))

    def param_specs(self):
        k = self.kernelSize
        fan_in = self.nIn * k[0] * k[1]
        fan_out = self.nOut * k[0] * k[1] / (self.stride[0] * self.stride[1])
        s = []
        if self.hasBias:
            s.append(ParamSpec("b", (1, self.nOut), "c", "bias", fan_in, fan_out))
        s.append(ParamSpec("W", (self.nOut, self.nIn, k[0], k[1]), "c", "weight", fan_in, fan_out))
        return s

    def forward(self, p, x, training, mask=None, ctx=None, skip_bias=False):
        """``skip_bias``: the graph executor hands the bias to the batch norm that follows (see its ``pre_bias``)."""
        x = self.apply_dropout(x, training)
        p = self.noisy(p, training)
        nhwc = self.cnn2dDataFormat == CNN2DFormat.NHWC
        if nhwc:
            x = x.permute(0, 3, 1, 2)
        if tuple(self.kernelSize) == (1, 1) and tuple(self.padding) == (0, 0) and x.is_cuda and type(self) is ConvolutionLayer:
            # pointwise convolution = GEMM over the channels-last activation: runs on the tcgen05 kernel
            from ...ops import native as nat
            from ...ops import nnops
            if not nnops._FORCE_TORCH:
                z = nat.conv1x1(x, p["W"], p["b"] if self.hasBias and not skip_bias else None, tuple(self.stride))
                if z is not None:
                    z = self.activation(z, training)
                    return z.permute(0, 2, 3, 1) if nhwc else z
        W = None
        if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and type(self) is ConvolutionLayer \
                and tuple(self.stride) == (1, 1) and x.shape[1] % 8 == 0 and self.nOut % 8 == 0:
            # stride-1 convolution of any kernel size: tcgen05 implicit GEMM (forward, dgrad, wgrad), no library convolution
            from ...ops import native as nat
            from ...ops import nnops as _nn
            if not _nn._FORCE_TORCH and nat.available():
                xp, pad = _pad_for_mode(x, self.kernelSize, self.stride, self.padding, self.dilation, self._mode())
                z = nat.conv2d(xp, p["W"], p["b"] if self.hasBias and not skip_bias else None, pad, self.dilation)
                if z is not None:
                    z = self.activation(z, training)
                    return z.permute(0, 2, 3, 1) if nhwc else z
        if x.is_cuda and x.dtype == torch.bfloat16 and type(self) is ConvolutionLayer:
            from ...ops import native as nat
            from ...ops import nnops as _nn
            if not _nn._FORCE_TORCH:
                W = nat.conv_weight_cl(p["W"])          # cast + channels-last relayout in one pass, gradient added in place
        if W is None:
            W = p["W"].to(x.dtype) if p["W"].dtype != x.dtype else p["W"]
        b = p["b"].reshape(-1).to(x.dtype) if self.hasBias and not skip_bias else None
        x, pad = _pad_for_mode(x, self.kernelSize, self.stride, self.padding, self.dilation, self._mode())
        if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and x.shape[1] < 8 and x.dim() == 4:
            if tuple(self.stride) == (2, 2) and tuple(self.dilation) == (1, 1) and x.shape[1] <= 4:
                z = _stem_space_to_depth(x, W, b, tuple(self.kernelSize), tuple(pad))
                z = self.activation(z, training)
                return z.permute(0, 2, 3, 1) if nhwc else z
            # an RGB stem has too few input channels for the tensor-core convolution kernels: zero-pad them to 8
            extra = 8 - x.shape[1]
            x = F.pad(x, (0, 0, 0, 0, 0, extra)).contiguous(memory_format=torch.channels_last)
            W = F.pad(W, (0, 0, 0, 0, 0, extra))
        z = nnops_conv2d(x, W, b, self.stride, pad, self.dilation)
        z = self.activation(z, training)
        return z.permute(0, 2, 3, 1) if nhwc else z


Convolution2D = ConvolutionLayer


def _stem_space_to_depth(x, W, b, k, pad):
    """Stride-2 convolution over a few input channels (an RGB stem) rewritten as a stride-1 convolution over a 2x2
    space-to-depth view: ``y[oh] = sum_kh W[kh] x[2 oh + kh]`` with ``kh = 2 a + bh`` becomes
    ``sum_a sum_bh W'[bh][a] x'[bh][oh + a]``.  The rewritten problem has 4x the channels (padded to 16) and half the
    taps per axis, which the tensor-core convolution kernels handle well; the 3-channel original does not."""
    N, C, H, Wd = x.shape
    kH, kW = k
    OH, OW = (H + 2 * pad[0] - kH) // 2 + 1, (Wd + 2 * pad[1] - kW) // 2 + 1
    KH2, KW2 = (kH + 1) // 2, (kW + 1) // 2
    Hs, Ws = OH + KH2 - 1, OW + KW2 - 1                    # space-to-depth extent the stride-1 convolution needs
    W8 = F.pad(W, (0, 2 * KW2 - kW, 0, 2 * KH2 - kH))
    Wsd = W8.reshape(W.shape[0], C, KH2, 2, KW2, 2).permute(0, 3, 5, 1, 2, 4).reshape(W.shape[0], 4 * C, KH2, KW2)
    cpad = (-4 * C) % 8
    if cpad:
        Wsd = F.pad(Wsd, (0, 0, 0, 0, 0, cpad))
    xs = None
    if x.is_cuda and not x.requires_grad and not nnops._FORCE_TORCH:
        from ...ops import native as nat
        xs = nat.stem_space_to_depth(x, pad, Hs, Ws, 4 * C + cpad)      # one kernel: padded 2x2 view, channels-last, padded channels
    if xs is None:
        eh, ew = 2 * Hs - (H + 2 * pad[0]), 2 * Ws - (Wd + 2 * pad[1])
        xp = F.pad(x, (pad[1], pad[1] + max(ew, 0), pad[0], pad[0] + max(eh, 0)))[:, :, :2 * Hs, :2 * Ws]
        xs = xp.reshape(N, C, Hs, 2, Ws, 2).permute(0, 3, 5, 1, 2, 4).reshape(N, 4 * C, Hs, Ws)
        if cpad:
            xs = F.pad(xs, (0, 0, 0, 0, 0, cpad))
        xs = xs.contiguous(memory_format=torch.channels_last)
    if xs.is_cuda and not nnops._FORCE_TORCH and xs.shape[1] % 8 == 0 and Wsd.shape[0] % 8 == 0:
        # stride-1 convolution over the space-to-depth view on the native kernels; the KW2 taps of a filter row times the
        # padded channels are one 64-element run per output pixel, loaded as a single K slice
        from ...ops import native as nat
        z = nat.conv2d(xs, Wsd, b, (0, 0), (1, 1), fuse_w=True)
        if z is not None:
            return z
    return F.conv2d(xs, Wsd, b)


def nnops_conv2d(x, W, b, stride, pad, dilation, groups=1):
    if x.is_cuda and not torch.backends.cudnn.benchmark:
        # the layers' default ``cudnnAlgoMode = PREFER_FASTEST``: let cuDNN time its algorithms once per shape
        torch.backends.cudnn.benchmark = True
    return F.conv2d(x, W, b, stride=tuple(stride), padding=tuple(pad), dilation=tuple(dilation), groups=groups)


class Convolution1DLayer(ConvolutionLayer):
    """1-D convolution over [mb, nIn, T]; parameters stored as 2-D kernels [nOut,nIn,k,1]."""
    JAVA_CLASS = _L + "Convolution1DLayer"
    DEFAULTS = {"rnnDataFormat": RNNFormat.NCW, "kernelSize": [5], "stride": [1], "padding": [0], "dilation": [1]}
    ND = 1

    def setNIn(self, it, override):
        if not self.nIn or override:
            self.nIn = it.size

    def preprocessor_for(self, it):
        return None

    def output_type(self, it):
        t = it.timeSeriesLength
        if t and t > 0:
            t = conv_out_size(t, self.kernelSize[0], self.stride[0], self.padding[0], self.dilation[0], self._mode())
        return InputType.recurrent(self.nOut, t, self.rnnDataFormat)

    def param_specs(self):
        k = self.kernelSize[0]
        fan_in, fan_out = self.nIn * k, self.nOut * k / self.stride[0]
        s = []
        if self.hasBias:
            s.append(ParamSpec("b", (1, self.nOut), "c", "bias", fan_in, fan_out))
        s.append(ParamSpec("W", (self.nOut, self.nIn, k, 1), "c", "weight", fan_in, fan_out))
        return s

    def forward(self, p, x, training, mask=None, ctx=None):
        x = self.apply_dropout(x, training)
        if self.rnnDataFormat == RNNFormat.NWC:
            x = x.permute(0, 2, 1)
        W = p["W"][..., 0].to(x.dtype)
        b = p["b"].reshape(-1).to(x.dtype) if self.hasBias else None
        x, pad = _pad_for_mode(x, self.kernelSize, self.stride, self.padding, self.dilation, self._mode())
        z = F.conv1d(x, W, b, stride=self.stride[0], padding=pad[0], dilation=self.dilation[0])
        z = self.activation(z, training)
        return z.permute(0, 2, 1) if self.rnnDataFormat == RNNFormat.NWC else z

    def feed_forward_mask(self, mask, input_type=None):
        if mask is None or self.stride[0] == 1 and self._mode() in (ConvolutionMode.Same, ConvolutionMode.Causal):
            return mask
        t_out = conv_out_size(mask.shape[1], self.kernelSize[0], self.stride[0], self.padding[0], self.dilation[0], self._mode())
        return F.adaptive_max_pool1d(mask.unsqueeze(1).float(), t_out).squeeze(1).to(mask.dtype)


Convolution1D = Convolution1DLayer


class Convolution3D(ConvolutionLayer):
    JAVA_CLASS = _L + "Convolution3D"
    DEFAULTS = {"dataFormat": "NCDHW", "kernelSize": [2, 2, 2], "stride": [1, 1, 1], "padding": [0, 0, 0], "dilation": [1, 1, 1]}
    ND = 3

    def preprocessor_for(self, it):
        return None

    def output_type(self, it):
        dims = [conv_out_size(getattr(it, n), self.kernelSize[i], self.stride[i], self.padding[i], self.dilation[i], self._mode())
                for i, n in enumerate(("depth", "height", "width"))]
        return InputType.convolutional3D(dims[0], dims[1], dims[2], self.nOut, self.dataFormat)

    def param_specs(self):
        k = self.kernelSize
        vol = k[0] * k[1] * k[2]
        fan_in, fan_out = self.nIn * vol, self.nOut * vol / (self.stride[0] * self.stride[1] * self.stride[2])
        s = []
        if self.hasBias:
            s.append(ParamSpec("b", (1, self.nOut), "c", "bias", fan_in, fan_out))
        s.append(ParamSpec("W", (self.nOut, self.nIn, k[0], k[1], k[2]), "c", "weight", fan_in, fan_out))
        return s

    def forward(self, p, x, training, mask=None, ctx=None):
        x = self.apply_dropout(x, training)
        ndhwc = self.dataFormat == "NDHWC"
        if ndhwc:
            x = x.permute(0, 4, 1, 2, 3)
        x, pad = _pad_for_mode(x, self.kernelSize, self.stride, self.padding, self.dilation, self._mode())
        z = F.conv3d(x, p["W"].to(x.dtype), p["b"].reshape(-1).to(x.dtype) if self.hasBias else None,
                     stride=tuple(self.stride), padding=tuple(pad), dilation=tuple(self.dilation))
        z = self.activation(z, training)
        return z.permute(0, 2, 3, 4, 1) if ndhwc else z


class Deconvolution2D(ConvolutionLayer):
    """Transposed convolution; weights ``[nIn, nOut, kH, kW]`` (``DeconvolutionParamInitializer``)."""
    JAVA_CLASS = _L + "Deconvolution2D"

    def output_type(self, it):
        def o(size, i):
            if self._mode() == ConvolutionMode.Same:
                return size * self.stride[i]
            return self.stride[i] * (size - 1) + (self.kernelSize[i] - 1) * self.dilation[i] + 1 - 2 * self.padding[i]
        return InputType.convolutional(o(it.height, 0), o(it.width, 1), self.nOut, getattr(it, "format", CNN2DFormat.NCHW))

    def param_specs(self):
        k = self.kernelSize
        fan_in, fan_out = self.nIn * k[0] * k[1], self.nOut * k[0] * k[1]
        s = []
        if self.hasBias:
            s.append(ParamSpec("b", (1, self.nOut), "c", "bias", fan_in, fan_out))
        s.append(ParamSpec("W", (self.nIn, self.nOut, k[0], k[1]), "c", "weight", fan_in, fan_out))
        return s

    def forward(self, p, x, training, mask=None, ctx=None):
        x = self.apply_dropout(x, training)
        b = p["b"].reshape(-1).to(x.dtype) if self.hasBias else None
        if self._mode() == ConvolutionMode.Same:
            z = F.conv_transpose2d(x, p["W"].to(x.dtype), b, stride=tuple(self.stride), padding=0, dilation=tuple(self.dilation))
            th, tw = x.shape[2] * self.stride[0], x.shape[3] * self.stride[1]
            oh, ow = (z.shape[2] - th) // 2, (z.shape[3] - tw) // 2
            z = z[:, :, oh:oh + th, ow:ow + tw]
        else:
            z = F.conv_transpose2d(x, p["W"].to(x.dtype), b, stride=tuple(self.stride), padding=tuple(self.padding),
                                   dilation=tuple(self.dilation))
        return self.activation(z, training)


class Deconvolution3D(Convolution3D):
    JAVA_CLASS = _L + "Deconvolution3D"

    def output_type(self, it):
        def o(size, i):
            if self._mode() == ConvolutionMode.Same:
                return size * self.stride[i]
            return self.stride[i] * (size - 1) + (self.kernelSize[i] - 1) * self.dilation[i] + 1 - 2 * self.padding[i]
        return InputType.convolutional3D(o(it.depth, 0), o(it.height, 1), o(it.width, 2), self.nOut, self.dataFormat)

    def param_specs(self):
        k = self.kernelSize
        vol = k[0] * k[1] * k[2]
        s = []
        if self.hasBias:
            s.append(ParamSpec("b", (1, self.nOut), "c", "bias", self.nIn * vol, self.nOut * vol))
        s.append(ParamSpec("W", (self.nIn, self.nOut, k[0], k[1], k[2]), "c", "weight", self.nIn * vol, self.nOut * vol))
        return s

    def forward(self, p, x, training, mask=None, ctx=None):
        x = self.apply_dropout(x, training)
        b = p["b"].reshape(-1).to(x.dtype) if self.hasBias else None
        pad = (0, 0, 0) if self._mode() == ConvolutionMode.Same else tuple(self.padding)
        z = F.conv_transpose3d(x, p["W"].to(x.dtype), b, stride=tuple(self.stride), padding=pad, dilation=tuple(self.dilation))
        if self._mode() == ConvolutionMode.Same:
            tgt = [x.shape[2 + i] * self.stride[i] for i in range(3)]
            off = [(z.shape[2 + i] - tgt[i]) // 2 for i in range(3)]
            z = z[:, :, off[0]:off[0] + tgt[0], off[1]:off[1] + tgt[1], off[2]:off[2] + tgt[2]]
        return self.activation(z, training)


class DepthwiseConvolution2D(ConvolutionLayer):
    JAVA_CLASS = _L + "DepthwiseConvolution2D"
    DEFAULTS = {"depthMultiplier": 1}

    def _finalise(self):
        super()._finalise()
        if self.nIn and not self.nOut:
            self.nOut = self.nIn * self.depthMultiplier

    def setNIn(self, it, override):
        super().setNIn(it, override)
        self.nOut = self.nIn * self.depthMultiplier

    def param_specs(self):
        k = self.kernelSize
        fan_in, fan_out = self.nIn * k[0] * k[1], self.depthMultiplier * k[0] * k[1]
        s = []
        if self.hasBias:
            s.append(ParamSpec("b", (1, self.nIn * self.depthMultiplier), "c", "bias", fan_in, fan_out))
        s.append(ParamSpec("W", (k[0], k[1], self.nIn, self.depthMultiplier), "c", "weight", fan_in, fan_out))
        return s

    def forward(self, p, x, training, mask=None, ctx=None):
        x = self.apply_dropout(x, training)
        k = self.kernelSize
        W = p["W"].permute(2, 3, 0, 1).reshape(self.nIn * self.depthMultiplier, 1, k[0], k[1]).to(x.dtype)
        b = p["b"].reshape(-1).to(x.dtype) if self.hasBias else None
        x, pad = _pad_for_mode(x, self.kernelSize, self.stride, self.padding, self.dilation, self._mode())
        return self.activation(nnops_conv2d(x, W, b, self.stride, pad, self.dilation, groups=self.nIn), training)


class SeparableConvolution2D(ConvolutionLayer):
    JAVA_CLASS = _L + "SeparableConvolution2D"
    DEFAULTS = {"depthMultiplier": 1}

    def param_specs(self):
        k = self.kernelSize
        fan_in, fan_out = self.nIn * k[0] * k[1], self.nOut * k[0] * k[1]
        s = []
        if self.hasBias:
            s.append(ParamSpec("b", (1, self.nOut), "c", "bias", fan_in, fan_out))
        s.append(ParamSpec("W", (self.depthMultiplier, self.nIn, k[0], k[1]), "c", "weight", fan_in, fan_out))
        s.append(ParamSpec("pW", (self.nOut, self.nIn * self.depthMultiplier, 1, 1), "c", "weight", fan_in, fan_out))
        return s

    def forward(self, p, x, training, mask=None, ctx=None):
        x = self.apply_dropout(x, training)
        k = self.kernelSize
        dW = p["W"].permute(1, 0, 2, 3).reshape(self.nIn * self.depthMultiplier, 1, k[0], k[1]).to(x.dtype)
        x, pad = _pad_for_mode(x, self.kernelSize, self.stride, self.padding, self.dilation, self._mode())
        z = nnops_conv2d(x, dW, None, self.stride, pad, self.dilation, groups=self.nIn)
        z = F.conv2d(z, p["pW"].to(x.dtype), p["b"].reshape(-1).to(x.dtype) if self.hasBias else None)
        return self.activation(z, training)


# --------------------------------------------------------------------------- pooling
class SubsamplingLayer(NoParamLayer):
    JAVA_CLASS = _L + "SubsamplingLayer"
    DEFAULTS = {"convolutionMode": None, "poolingType": PoolingType.MAX, "kernelSize": [1, 1], "stride": [2, 2],
                "padding": [0, 0], "dilation": [1, 1], "pnorm": 0, "eps": 1e-8, "cudnnAllowFallback": True,
                "cnn2dDataFormat": CNN2DFormat.NCHW, "avgPoolIncludePadInDivisor": True}
    INHERIT = ("convolutionMode",)
    ND = 2

    def _positional(self, *args):
        names = ("poolingType", "kernelSize", "stride", "padding")
        if args and not isinstance(args[0], str):
            names = names[1:]
        for n, a in zip(names, args):
            setattr(self, n, a)
            self._explicit.add(n)

    def _finalise(self):
        super()._finalise()
        for f in ("kernelSize", "stride", "padding", "dilation"):
            setattr(self, f, _pair(getattr(self, f), self.ND))
        self.poolingType = str(self.poolingType).upper()

    def _mode(self):
        return self.convolutionMode or ConvolutionMode.Truncate

    def preprocessor_for(self, it):
        from ..conf.preprocessors import FeedForwardToCnnPreProcessor
        if it.kind == InputType.CNNFlat:
            return FeedForwardToCnnPreProcessor(it.height, it.width, it.channels)
        return None

    def output_type(self, it):
        h = conv_out_size(it.height, self.kernelSize[0], self.stride[0], self.padding[0], self.dilation[0], self._mode())
        w = conv_out_size(it.width, self.kernelSize[1], self.stride[1], self.padding[1], self.dilation[1], self._mode())
        return InputType.convolutional(h, w, it.channels, getattr(it, "format", CNN2DFormat.NCHW))

    def _pool(self, x, pad):
        k, s, d = tuple(self.kernelSize), tuple(self.stride), tuple(self.dilation)
        fns = {1: (F.max_pool1d, F.avg_pool1d, F.lp_pool1d), 2: (F.max_pool2d, F.avg_pool2d, F.lp_pool2d),
               3: (F.max_pool3d, F.avg_pool3d, getattr(F, "lp_pool3d", None))}[self.ND]
        if self.poolingType == PoolingType.MAX:
            if self.ND == 2 and x.is_cuda and d == (1, 1):
                from ...ops import native as nat
                from ...ops import nnops
                z = None if nnops._FORCE_TORCH else nat.maxpool2d(x, k, s, tuple(pad))
                if z is not None:
                    return z
            return fns[0](x, k, s, tuple(pad), d)
        if self.poolingType == PoolingType.AVG:
            return fns[1](x, k, s, tuple(pad), count_include_pad=self.avgPoolIncludePadInDivisor)
        if self.poolingType == PoolingType.SUM:
            n = 1
            for e in k:
                n *= e
            return fns[1](x, k, s, tuple(pad), count_include_pad=True) * n
        if self.poolingType == PoolingType.PNORM:
            n = 1
            for e in k:
                n *= e
            pw = fns[1](x.abs() ** self.pnorm, k, s, tuple(pad), count_include_pad=True) * n
            return pw ** (1.0 / self.pnorm)
        raise ValueError(self.poolingType)

    def forward(self, p, x, training, mask=None, ctx=None):
        nhwc = self.ND == 2 and self.cnn2dDataFormat == CNN2DFormat.NHWC
        if nhwc:
            x = x.permute(0, 3, 1, 2)
        fill = float("-inf") if self.poolingType == PoolingType.MAX else 0.0
        x, pad = _pad_for_mode(x, self.kernelSize, self.stride, self.padding, self.dilation, self._mode(), value=fill)
        z = self._pool(x, pad)
        return z.permute(0, 2, 3, 1) if nhwc else z


Pooling2D = SubsamplingLayer


class Subsampling1DLayer(SubsamplingLayer):
    JAVA_CLASS = _L + "Subsampling1DLayer"
    DEFAULTS = {"kernelSize": [2], "stride": [2], "padding": [0], "dilation": [1]}
    ND = 1

    def preprocessor_for(self, it):
        return None

    def output_type(self, it):
        t = it.timeSeriesLength
        if t and t > 0:
            t = conv_out_size(t, self.kernelSize[0], self.stride[0], self.padding[0], self.dilation[0], self._mode())
        return InputType.recurrent(it.size, t, getattr(it, "format", RNNFormat.NCW))


Pooling1D = Subsampling1DLayer


class Subsampling3DLayer(SubsamplingLayer):
    JAVA_CLASS = _L + "Subsampling3DLayer"
    DEFAULTS = {"kernelSize": [1, 1, 1], "stride": [2, 2, 2], "padding": [0, 0, 0], "dilation": [1, 1, 1], "dataFormat": "NCDHW"}
    ND = 3

    def preprocessor_for(self, it):
        return None

    def output_type(self, it):
        dims = [conv_out_size(getattr(it, n), self.kernelSize[i], self.stride[i], self.padding[i], self.dilation[i], self._mode())
                for i, n in enumerate(("depth", "height", "width"))]
        return InputType.convolutional3D(dims[0], dims[1], dims[2], it.channels, self.dataFormat)


class GlobalPoolingLayer(NoParamLayer):
    JAVA_CLASS = _L + "GlobalPoolingLayer"
    DEFAULTS = {"poolingType": PoolingType.MAX, "poolingDimensions": None, "pnorm": 2, "collapseDimensions": True}

    def _positional(self, *args):
        if args:
            self.poolingType = args[0]

    def _finalise(self):
        super()._finalise()
        self.poolingType = str(self.poolingType).upper()

    def output_type(self, it):
        if it.kind == InputType.RNN:
            return InputType.feedForward(it.size)
        if it.kind in (InputType.CNN, InputType.CNN3D):
            return InputType.feedForward(it.channels)
        return it

    def forward(self, p, x, training, mask=None, ctx=None):
        dims = self.poolingDimensions or list(range(2, x.dim()))
        dims = tuple(dims)
        if mask is not None and x.dim() == 3:
            m = mask.unsqueeze(1).to(x.dtype)
            if self.poolingType == PoolingType.MAX:
                z = (x.masked_fill(m == 0, float("-inf"))).amax(dim=dims, keepdim=not self.collapseDimensions)
            elif self.poolingType == PoolingType.AVG:
                z = (x * m).sum(dims, keepdim=not self.collapseDimensions) / m.sum(dims, keepdim=not self.collapseDimensions).clamp_min(1)
            elif self.poolingType == PoolingType.SUM:
                z = (x * m).sum(dims, keepdim=not self.collapseDimensions)
            else:
                z = ((x * m).abs() ** self.pnorm).sum(dims, keepdim=not self.collapseDimensions) ** (1.0 / self.pnorm)
            return z
        kd = not self.collapseDimensions
        if self.poolingType == PoolingType.MAX:
            return x.amax(dim=dims, keepdim=kd)
        if self.poolingType == PoolingType.AVG:
            return x.mean(dim=dims, keepdim=kd)
        if self.poolingType == PoolingType.SUM:
            return x.sum(dim=dims, keepdim=kd)
        return (x.abs() ** self.pnorm).sum(dim=dims, keepdim=kd) ** (1.0 / self.pnorm)

    def feed_forward_mask(self, mask, input_type=None):
        return None


# --------------------------------------------------------------------------- padding / cropping / upsampling
class ZeroPaddingLayer(NoParamLayer):
    JAVA_CLASS = _L + "ZeroPaddingLayer"
    DEFAULTS = {"padding": [0, 0, 0, 0], "dataFormat": CNN2DFormat.NCHW}   # top, bottom, left, right

    def _positional(self, *args):
        if len(args) == 1:
            args = args[0] if isinstance(args[0], (list, tuple)) else (args[0], args[0])
        if len(args) == 2:
            self.padding = [args[0], args[0], args[1], args[1]]
        elif len(args) == 4:
            self.padding = list(args)

    def output_type(self, it):
        p = self.padding
        return InputType.convolutional(it.height + p[0] + p[1], it.width + p[2] + p[3], it.channels, getattr(it, "format", CNN2DFormat.NCHW))

    def forward(self, p, x, training, mask=None, ctx=None):
        t, b, l, r = self.padding
        if self.dataFormat == CNN2DFormat.NHWC:
            return F.pad(x, [0, 0, l, r, t, b])
        return F.pad(x, [l, r, t, b])


class ZeroPadding1DLayer(NoParamLayer):
    JAVA_CLASS = _L + "ZeroPadding1DLayer"
    DEFAULTS = {"padding": [0, 0]}

    def _positional(self, *args):
        if len(args) == 1:
            self.padding = [args[0], args[0]] if isinstance(args[0], int) else list(args[0])
        elif len(args) == 2:
            self.padding = list(args)

    def output_type(self, it):
        t = it.timeSeriesLength
        return InputType.recurrent(it.size, t + sum(self.padding) if t and t > 0 else t, getattr(it, "format", RNNFormat.NCW))

    def forward(self, p, x, training, mask=None, ctx=None):
        return F.pad(x, list(self.padding))


class ZeroPadding3DLayer(NoParamLayer):
    JAVA_CLASS = _L + "ZeroPadding3DLayer"
    DEFAULTS = {"padding": [0, 0, 0, 0, 0, 0]}   # d-, d+, h-, h+, w-, w+

    def _positional(self, *args):
        if len(args) == 1:
            args = (args[0],) * 3 if isinstance(args[0], int) else tuple(args[0])
        if len(args) == 3:
            self.padding = [args[0], args[0], args[1], args[1], args[2], args[2]]
        elif len(args) == 6:
            self.padding = list(args)

    def output_type(self, it):
        p = self.padding
        return InputType.convolutional3D(it.depth + p[0] + p[1], it.height + p[2] + p[3], it.width + p[4] + p[5], it.channels)

    def forward(self, p, x, training, mask=None, ctx=None):
        d0, d1, h0, h1, w0, w1 = self.padding
        return F.pad(x, [w0, w1, h0, h1, d0, d1])


class Cropping2D(NoParamLayer):
    JAVA_CLASS = _L + "convolutional.Cropping2D"
    DEFAULTS = {"cropping": [0, 0, 0, 0], "dataFormat": CNN2DFormat.NCHW}

    def _positional(self, *args):
        if len(args) == 2:
            self.cropping = [args[0], args[0], args[1], args[1]]
        elif len(args) == 4:
            self.cropping = list(args)
        elif len(args) == 1:
            a = args[0]
            self.cropping = [a, a, a, a] if isinstance(a, int) else list(a)

    def output_type(self, it):
        c = self.cropping
        return InputType.convolutional(it.height - c[0] - c[1], it.width - c[2] - c[3], it.channels, getattr(it, "format", CNN2DFormat.NCHW))

    def forward(self, p, x, training, mask=None, ctx=None):
        t, b, l, r = self.cropping
        if self.dataFormat == CNN2DFormat.NHWC:
            return x[:, t:x.shape[1] - b, l:x.shape[2] - r, :]
        return x[:, :, t:x.shape[2] - b, l:x.shape[3] - r]


class Cropping1D(NoParamLayer):
    JAVA_CLASS = _L + "convolutional.Cropping1D"
    DEFAULTS = {"cropping": [0, 0]}

    def _positional(self, *args):
        if len(args) == 1:
            self.cropping = [args[0], args[0]] if isinstance(args[0], int) else list(args[0])
        elif len(args) == 2:
            self.cropping = list(args)

    def output_type(self, it):
        t = it.timeSeriesLength
        return InputType.recurrent(it.size, t - sum(self.cropping) if t and t > 0 else t, getattr(it, "format", RNNFormat.NCW))

    def forward(self, p, x, training, mask=None, ctx=None):
        return x[:, :, self.cropping[0]:x.shape[2] - self.cropping[1]]


class Cropping3D(NoParamLayer):
    JAVA_CLASS = _L + "convolutional.Cropping3D"
    DEFAULTS = {"cropping": [0, 0, 0, 0, 0, 0]}

    def _positional(self, *args):
        if len(args) == 3:
            self.cropping = [args[0], args[0], args[1], args[1], args[2], args[2]]
        elif len(args) == 6:
            self.cropping = list(args)

    def output_type(self, it):
        c = self.cropping
        return InputType.convolutional3D(it.depth - c[0] - c[1], it.height - c[2] - c[3], it.width - c[4] - c[5], it.channels)

    def forward(self, p, x, training, mask=None, ctx=None):
        c = self.cropping
        return x[:, :, c[0]:x.shape[2] - c[1], c[2]:x.shape[3] - c[3], c[4]:x.shape[4] - c[5]]


class Upsampling2D(NoParamLayer):
    JAVA_CLASS = _L + "Upsampling2D"
    DEFAULTS = {"size": [2, 2], "format": CNN2DFormat.NCHW}

    def _positional(self, *args):
        if args:
            self.size = args[0]

    def _finalise(self):
        super()._finalise()
        self.size = _pair(self.size, 2)

    def output_type(self, it):
        return InputType.convolutional(it.height * self.size[0], it.width * self.size[1], it.channels, getattr(it, "format", CNN2DFormat.NCHW))

    def forward(self, p, x, training, mask=None, ctx=None):
        if self.format == CNN2DFormat.NHWC:
            return x.repeat_interleave(self.size[0], 1).repeat_interleave(self.size[1], 2)
        return x.repeat_interleave(self.size[0], 2).repeat_interleave(self.size[1], 3)


class Upsampling1D(NoParamLayer):
    JAVA_CLASS = _L + "Upsampling1D"
    DEFAULTS = {"size": [2]}

    def _positional(self, *args):
        if args:
            self.size = args[0]

    def _finalise(self):
        super()._finalise()
        self.size = _pair(self.size, 1)

    def output_type(self, it):
        t = it.timeSeriesLength
        return InputType.recurrent(it.size, t * self.size[0] if t and t > 0 else t, getattr(it, "format", RNNFormat.NCW))

    def forward(self, p, x, training, mask=None, ctx=None):
        return x.repeat_interleave(self.size[0], 2)


class Upsampling3D(NoParamLayer):
    JAVA_CLASS = _L + "Upsampling3D"
    DEFAULTS = {"size": [2, 2, 2], "dataFormat": "NCDHW"}

    def _positional(self, *args):
        if args:
            self.size = args[0]

    def _finalise(self):
        super()._finalise()
        self.size = _pair(self.size, 3)

    def output_type(self, it):
        return InputType.convolutional3D(it.depth * self.size[0], it.height * self.size[1], it.width * self.size[2], it.channels)

    def forward(self, p, x, training, mask=None, ctx=None):
        return x.repeat_interleave(self.size[0], 2).repeat_interleave(self.size[1], 3).repeat_interleave(self.size[2], 4)


class SpaceToDepthLayer(NoParamLayer):
    JAVA_CLASS = _L + "SpaceToDepthLayer"
    DEFAULTS = {"blockSize": 2, "dataFormat": CNN2DFormat.NCHW}

    def _positional(self, *args):
        if args:
            self.blockSize = args[0]

    def output_type(self, it):
        b = self.blockSize
        return InputType.convolutional(it.height // b, it.width // b, it.channels * b * b, getattr(it, "format", CNN2DFormat.NCHW))

    def forward(self, p, x, training, mask=None, ctx=None):
        b = self.blockSize
        n, c, h, w = x.shape
        x = x.reshape(n, c, h // b, b, w // b, b).permute(0, 3, 5, 1, 2, 4)
        return x.reshape(n, c * b * b, h // b, w // b)


class SpaceToBatchLayer(NoParamLayer):
    JAVA_CLASS = _L + "SpaceToBatchLayer"
    DEFAULTS = {"blocks": [2, 2], "padding": [[0, 0], [0, 0]], "format": CNN2DFormat.NCHW}

    def output_type(self, it):
        p, b = self.padding, self.blocks
        return InputType.convolutional((it.height + p[0][0] + p[0][1]) // b[0], (it.width + p[1][0] + p[1][1]) // b[1],
                                       it.channels, getattr(it, "format", CNN2DFormat.NCHW))

    def forward(self, p, x, training, mask=None, ctx=None):
        pd, b = self.padding, self.blocks
        x = F.pad(x, [pd[1][0], pd[1][1], pd[0][0], pd[0][1]])
        n, c, h, w = x.shape
        x = x.reshape(n, c, h // b[0], b[0], w // b[1], b[1]).permute(3, 5, 0, 1, 2, 4)
        return x.reshape(n * b[0] * b[1], c, h // b[0], w // b[1])


# --------------------------------------------------------------------------- normalisation
class BatchNormalization(FeedForwardLayer):
    JAVA_CLASS = _L + "BatchNormalization"
    DEFAULTS = {"decay": 0.9, "eps": 1e-5, "isMinibatch": True, "gamma": 1.0, "beta": 0.0, "lockGammaBeta": False,
                "cudnnAllowFallback": True, "useLogStd": True, "cnn2DFormat": CNN2DFormat.NCHW}

    def setNIn(self, it, override):
        if self.nIn and not override:
            self.nOut = self.nIn
            return
        if it.kind in (InputType.CNN, InputType.CNNFlat, InputType.CNN3D):
            self.nIn = it.channels
        else:
            self.nIn = it.size
        self.nOut = self.nIn

    def output_type(self, it):
        return it

    def preprocessor_for(self, it):
        from ..conf.preprocessors import FeedForwardToCnnPreProcessor
        if it.kind == InputType.CNNFlat:
            return FeedForwardToCnnPreProcessor(it.height, it.width, it.channels)
        return None

    def param_specs(self):
        n = self.nOut or self.nIn
        s = []
        if not self.lockGammaBeta:
            s.append(ParamSpec("gamma", (1, n), "c", "weight", n, n, init=self.gamma))
            s.append(ParamSpec("beta", (1, n), "c", "bias", n, n, init=self.beta))
        s.append(ParamSpec("mean", (1, n), "c", "state", n, n, init=0.0))
        s.append(ParamSpec("log10stdev" if self.useLogStd else "var", (1, n), "c", "state", n, n,
                           init=0.0 if self.useLogStd else 1.0))
        return s

    def regularizers(self, spec):
        return []   # the reference never regularises batch-norm parameters

    def forward(self, p, x, training, mask=None, ctx=None, fuse_relu=False, residual=None, pre_bias=None):
        """``fuse_relu`` / ``residual`` are set by the graph executor when this layer is followed by a ReLU (optionally
        after an element-wise add): the result is then ``relu(bn(x) [+ residual])`` from one fused kernel chain.
        ``pre_bias`` is the bias of the convolution that produced ``x`` when the executor left it out of ``x``: batch
        statistics cancel it in training (its gradient is exactly zero), so it only enters the running mean and the
        inference-time shift."""
        n = self.nOut or self.nIn
        nhwc = x.dim() == 4 and self.cnn2DFormat == CNN2DFormat.NHWC
        if nhwc:
            x = x.permute(0, 3, 1, 2)
            if residual is not None:
                residual = residual.permute(0, 3, 1, 2)
        if self.lockGammaBeta:
            g = torch.full((n,), self.gamma, device=x.device, dtype=torch.float32)
            b = torch.full((n,), self.beta, device=x.device, dtype=torch.float32)
        else:
            g, b = p["gamma"].reshape(-1), p["beta"].reshape(-1)
        mean = p["mean"].reshape(-1)
        if self.useLogStd:
            sv = p["log10stdev"].reshape(-1)
        else:
            sv = p["var"].reshape(-1)
        from ...ops import native as nat
        from ...ops import nnops
        if not nnops._FORCE_TORCH and x.dim() in (2, 4) and mean.dtype == torch.float32 and nat.bn_supported(x):
            # hand-written channels-last kernels: statistics, running-stat update, normalise (+ add) (+ ReLU)
            if training:
                # the parameter leaves themselves (not reshaped views): the backward kernel then adds dgamma / dbeta straight into
                # their slices of the flat gradient buffer and autograd launches no accumulation kernels
                g_leaf, b_leaf = (g, b) if self.lockGammaBeta else (p["gamma"], p["beta"])
                y = nat.bn_act_train(x, residual, g_leaf, b_leaf, mean.detach(), sv.detach(), self.useLogStd, self.decay, self.eps,
                                     fuse_relu, pre_bias)
            else:
                with torch.no_grad():
                    var = torch.pow(10.0, 2.0 * sv) if self.useLogStd else sv
                    scale = g.float() * torch.rsqrt(var + self.eps)
                    shift = b.float() - mean * scale
                    if pre_bias is not None:
                        shift = shift + pre_bias.reshape(-1).float() * scale
                y = nat.bn_act_eval(x, residual, scale, shift, fuse_relu)
            return y.permute(0, 2, 3, 1) if nhwc else y
        if pre_bias is not None:
            x = x + pre_bias.reshape(1, -1, *([1] * (x.dim() - 2))).to(x.dtype)
        var = torch.pow(10.0, 2.0 * sv.detach()) if self.useLogStd else sv.detach()
        if training:
            # batch statistics; running stats use DL4J's decay: global = decay*global + (1-decay)*batch
            rm, rv = mean.detach().clone(), var.clone()
            y = F.batch_norm(x, rm, rv, g.to(x.dtype) if x.dtype != g.dtype and x.dtype == torch.float64 else g,
                             b, True, 1.0 - self.decay, self.eps)
            with torch.no_grad():
                # F.batch_norm stores the *unbiased* variance; DL4J keeps the biased batch variance
                cnt = x.numel() / x.shape[1]
                if cnt > 1:
                    rv_b = (rv - self.decay * var) * ((cnt - 1.0) / cnt) + self.decay * var
                else:
                    rv_b = rv
                mean.data.copy_(rm)          # .data: no version bump on the shared flat buffer
                if self.useLogStd:
                    sv.data.copy_(0.5 * torch.log10(rv_b.clamp_min(1e-30)))
                else:
                    sv.data.copy_(rv_b)
        else:
            y = F.batch_norm(x, mean.detach(), var, g, b, False, 0.0, self.eps)
        # no activation of its own: the reference layer applies the normalisation only (its activationFn is never used)
        if residual is not None:
            y = y + residual
        if fuse_relu:
            y = torch.relu(y)
        return y.permute(0, 2, 3, 1) if nhwc else y


class LocalResponseNormalization(NoParamLayer):
    JAVA_CLASS = _L + "LocalResponseNormalization"
    DEFAULTS = {"n": 5.0, "k": 2.0, "beta": 0.75, "alpha": 1e-4, "cudnnAllowFallback": True, "dataFormat": CNN2DFormat.NCHW}

    def forward(self, p, x, training, mask=None, ctx=None):
        # DL4J: x / (k + alpha * sum_{window} x^2)^beta  (alpha is NOT divided by n)
        n = int(self.n)
        return F.local_response_norm(x, n, alpha=self.alpha * n, beta=self.beta, k=self.k)
