"""DataSet normalizers / pre-processors and ``NormalizerSerializer``.

Parity: ``nd4j-api/.../dataset/api/preprocessor`` (``NormalizerStandardize``, ``NormalizerMinMaxScaler``,
``ImagePreProcessingScaler``, ``VGG16ImagePreProcessor``, ``MultiNormalizer*``, composite / lambda
pre-processors) and ``.../preprocessor/serializer`` (stream layout: ``writeUTF("NORMALIZER")``,
``writeInt(1)``, ``writeUTF(type)``, then the strategy payload built from booleans, doubles and
``Nd4j.write`` arrays).  Statistics are accumulated in float64 on the data's device, one pass.
"""
from __future__ import annotations

import io
import struct

import torch

from ..nd.ndarray import INDArray
from ..serde import binary


def _t(x):
    if x is None:
        return None
    return x.t if isinstance(x, INDArray) else (x if isinstance(x, torch.Tensor) else torch.as_tensor(x))


def _feature_axes(x):
    """Axes reduced when computing per-feature statistics: everything except the feature/channel axis (1)."""
    return [0] + list(range(2, x.dim()))


def _bshape(x, stat):
    s = [1] * x.dim()
    s[1 if x.dim() > 1 else 0] = -1
    return stat.reshape(s)


class _RunningStats:
    def __init__(self):
        self.n = 0
        self.sum = self.sumsq = self.min = self.max = None

    def add(self, x, mask=None):
        x = x.double()
        ax = _feature_axes(x)
        if mask is not None and x.dim() == 3:
            m = mask.double().unsqueeze(1)
            cnt = float(m.sum())
            xs = x * m
            big = torch.finfo(torch.float64).max
            mn = torch.where(m > 0, x, torch.full_like(x, big)).amin(ax)
            mx = torch.where(m > 0, x, torch.full_like(x, -big)).amax(ax)
        else:
            cnt = float(x.numel() / x.shape[1]) if x.dim() > 1 else float(x.numel())
            xs, mn, mx = x, x.amin(ax), x.amax(ax)
        s, ss = xs.sum(ax).cpu(), (xs * xs).sum(ax).cpu()
        mn, mx = mn.cpu(), mx.cpu()
        if self.sum is None:
            self.sum, self.sumsq, self.min, self.max = s, ss, mn, mx
        else:
            self.sum += s
            self.sumsq += ss
            self.min, self.max = torch.minimum(self.min, mn), torch.maximum(self.max, mx)
        self.n += cnt

    def mean(self): return self.sum / self.n
    def std(self): return (self.sumsq / self.n - self.mean() ** 2).clamp(min=0).sqrt()


class DataNormalization:
    """Base: ``fit(DataSet | iterator)``, ``transform`` / ``preProcess``, ``revert``."""
    _fit_label = False

    def fitLabel(self, b=True): self._fit_label = bool(b); return self
    def isFitLabel(self): return self._fit_label

    def fit(self, data):
        fs, ls = _RunningStats(), _RunningStats()
        if hasattr(data, "getFeatures"):
            data = [data]
        elif hasattr(data, "reset"):
            data.reset()
        for ds in data:
            fs.add(_t(ds.getFeatures()), _t(ds.getFeaturesMaskArray()) if hasattr(ds, "getFeaturesMaskArray") else None)
            if self._fit_label and ds.getLabels() is not None:
                ls.add(_t(ds.getLabels()), _t(ds.getLabelsMaskArray()) if hasattr(ds, "getLabelsMaskArray") else None)
        self._set_stats(fs, ls if self._fit_label else None)
        return self

    def preProcess(self, ds):
        ds.setFeatures(self.transform(ds.getFeatures()))
        if self._fit_label and ds.getLabels() is not None:
            ds.setLabels(self.transformLabel(ds.getLabels()))
        return ds

    __call__ = preProcess

    def revert(self, ds):
        ds.setFeatures(self.revertFeatures(ds.getFeatures()))
        if self._fit_label and ds.getLabels() is not None:
            ds.setLabels(self.revertLabels(ds.getLabels()))
        return ds

    @staticmethod
    def _wrap(like, t):
        return INDArray(t) if isinstance(like, INDArray) else t


class NormalizerStandardize(DataNormalization):
    TYPE = "STANDARDIZE"

    def __init__(self, mean=None, std=None, labelMean=None, labelStd=None):
        self.mean_, self.std_ = _t(mean), _t(std)
        self.labelMean, self.labelStd = _t(labelMean), _t(labelStd)
        self._fit_label = labelMean is not None

    def _set_stats(self, fs, ls):
        self.mean_, self.std_ = fs.mean().float(), fs.std().float()
        if ls is not None:
            self.labelMean, self.labelStd = ls.mean().float(), ls.std().float()

    def getMean(self): return INDArray(self.mean_)
    def getStd(self): return INDArray(self.std_)
    def getLabelMean(self): return INDArray(self.labelMean)
    def getLabelStd(self): return INDArray(self.labelStd)

    @staticmethod
    def _fwd(x, m, s):
        xt = _t(x)
        s = torch.where(s == 0, torch.ones_like(s), s)            # constant columns: divide by 1 (reference adds eps)
        return (xt - _bshape(xt, m.to(xt.device, xt.dtype))) / _bshape(xt, s.to(xt.device, xt.dtype))

    @staticmethod
    def _bwd(x, m, s):
        xt = _t(x)
        s = torch.where(s == 0, torch.ones_like(s), s)
        return xt * _bshape(xt, s.to(xt.device, xt.dtype)) + _bshape(xt, m.to(xt.device, xt.dtype))

    def transform(self, x): return self._wrap(x, self._fwd(x, self.mean_, self.std_))
    def transformLabel(self, y): return self._wrap(y, self._fwd(y, self.labelMean, self.labelStd))
    def revertFeatures(self, x): return self._wrap(x, self._bwd(x, self.mean_, self.std_))
    def revertLabels(self, y): return self._wrap(y, self._bwd(y, self.labelMean, self.labelStd))


class NormalizerMinMaxScaler(DataNormalization):
    TYPE = "MIN_MAX"

    def __init__(self, minRange=0.0, maxRange=1.0):
        self.targetMin, self.targetMax = float(minRange), float(maxRange)
        self.min_ = self.max_ = self.labelMin = self.labelMax = None

    def _set_stats(self, fs, ls):
        self.min_, self.max_ = fs.min.float(), fs.max.float()
        if ls is not None:
            self.labelMin, self.labelMax = ls.min.float(), ls.max.float()

    def getMin(self): return INDArray(self.min_)
    def getMax(self): return INDArray(self.max_)
    def getLabelMin(self): return INDArray(self.labelMin)
    def getLabelMax(self): return INDArray(self.labelMax)
    def getTargetMin(self): return self.targetMin
    def getTargetMax(self): return self.targetMax

    def _fwd(self, x, mn, mx):
        xt = _t(x)
        rng = (mx - mn)
        rng = torch.where(rng == 0, torch.ones_like(rng), rng)
        z = (xt - _bshape(xt, mn.to(xt.device, xt.dtype))) / _bshape(xt, rng.to(xt.device, xt.dtype))
        return z * (self.targetMax - self.targetMin) + self.targetMin

    def _bwd(self, x, mn, mx):
        xt = _t(x)
        rng = (mx - mn)
        rng = torch.where(rng == 0, torch.ones_like(rng), rng)
        z = (xt - self.targetMin) / (self.targetMax - self.targetMin)
        return z * _bshape(xt, rng.to(xt.device, xt.dtype)) + _bshape(xt, mn.to(xt.device, xt.dtype))

    def transform(self, x): return self._wrap(x, self._fwd(x, self.min_, self.max_))
    def transformLabel(self, y): return self._wrap(y, self._fwd(y, self.labelMin, self.labelMax))
    def revertFeatures(self, x): return self._wrap(x, self._bwd(x, self.min_, self.max_))
    def revertLabels(self, y): return self._wrap(y, self._bwd(y, self.labelMin, self.labelMax))


class ImagePreProcessingScaler(DataNormalization):
    """Pixel values [0, maxPixelVal] -> [minRange, maxRange]; nothing to fit."""
    TYPE = "IMAGE_MIN_MAX"

    def __init__(self, minRange=0.0, maxRange=1.0, maxBits=8):
        self.minRange, self.maxRange = float(minRange), float(maxRange)
        self.maxPixelVal = float(2 ** maxBits - 1)

    def fit(self, data): return self
    def transform(self, x):
        xt = _t(x).float() if not _t(x).is_floating_point() else _t(x)
        return self._wrap(x, xt / self.maxPixelVal * (self.maxRange - self.minRange) + self.minRange)
    def revertFeatures(self, x):
        return self._wrap(x, (_t(x) - self.minRange) / (self.maxRange - self.minRange) * self.maxPixelVal)
    def transformLabel(self, y): return y
    def revertLabels(self, y): return y


class VGG16ImagePreProcessor(DataNormalization):
    """Subtracts the ImageNet channel means used by VGG16 (RGB 123.68, 116.779, 103.939)."""
    TYPE = "IMAGE_VGG16"
    VGG_MEAN_OFFSET_BGR = (123.68, 116.779, 103.939)

    def fit(self, data): return self
    def _m(self, xt): return torch.tensor(self.VGG_MEAN_OFFSET_BGR, dtype=xt.dtype, device=xt.device).reshape(1, 3, 1, 1)
    def transform(self, x): return self._wrap(x, _t(x) - self._m(_t(x)))
    def revertFeatures(self, x): return self._wrap(x, _t(x) + self._m(_t(x)))
    def transformLabel(self, y): return y
    def revertLabels(self, y): return y


class _MultiBase:
    """MultiDataSet variants: one underlying normalizer per input (and per output when fitLabel)."""
    UNDER = None

    def __init__(self, *a):
        self._args = a
        self.inputs, self.outputs = [], []
        self._fit_label = False

    def fitLabel(self, b=True): self._fit_label = bool(b); return self
    def isFitLabel(self): return self._fit_label
    def numInputs(self): return len(self.inputs)
    def numOutputs(self): return len(self.outputs)

    def fit(self, data):
        from .dataset import DataSet
        if hasattr(data, "getFeatures"):
            data = [data]
        elif hasattr(data, "reset"):
            data.reset()
        data = list(data)
        nf = len(data[0].getFeatures())
        self.inputs = [self.UNDER(*self._args) for _ in range(nf)]
        for i, n in enumerate(self.inputs):
            n.fit([DataSet(m.getFeatures()[i], None) for m in data])
        if self._fit_label:
            nl = len(data[0].getLabels())
            self.outputs = [self.UNDER(*self._args) for _ in range(nl)]
            for i, n in enumerate(self.outputs):
                n.fit([DataSet(m.getLabels()[i], None) for m in data])
        return self

    def preProcess(self, mds):
        mds.setFeatures([n.transform(f) for n, f in zip(self.inputs, mds.getFeatures())])
        if self._fit_label:
            mds.setLabels([n.transform(l) for n, l in zip(self.outputs, mds.getLabels())])
        return mds

    __call__ = preProcess

    def revert(self, mds):
        mds.setFeatures([n.revertFeatures(f) for n, f in zip(self.inputs, mds.getFeatures())])
        if self._fit_label:
            mds.setLabels([n.revertFeatures(l) for n, l in zip(self.outputs, mds.getLabels())])
        return mds


class MultiNormalizerStandardize(_MultiBase):
    TYPE, UNDER = "MULTI_STANDARDIZE", NormalizerStandardize


class MultiNormalizerMinMaxScaler(_MultiBase):
    TYPE, UNDER = "MULTI_MIN_MAX", NormalizerMinMaxScaler


class CompositeDataSetPreProcessor:
    def __init__(self, *pps, stopOnEmptyDataSet=False): self.pps, self.stop = list(pps), stopOnEmptyDataSet
    def preProcess(self, ds):
        for p in self.pps:
            if self.stop and ds.numExamples() == 0:
                return ds
            p.preProcess(ds)
        return ds
    __call__ = preProcess


class LambdaDataSetPreProcessor:
    def __init__(self, fn): self.fn = fn
    def preProcess(self, ds): self.fn(ds); return ds
    __call__ = preProcess


class LabelLastTimeStepPreProcessor:
    """[N, C, T] labels -> [N, C] taken at each example's last unmasked step."""
    def preProcess(self, ds):
        y = _t(ds.getLabels())
        m = _t(ds.getLabelsMaskArray())
        if m is None:
            ds.setLabels(y[:, :, -1])
        else:
            idx = (m > 0).long().cumsum(1).argmax(1)
            ds.setLabels(y[torch.arange(y.shape[0]), :, idx])
            ds.setLabelsMaskArray(None)
        return ds
    __call__ = preProcess


# ----------------------------------------------------------------------------- serializer
class NormalizerSerializer:
    HEADER = "NORMALIZER"

    @staticmethod
    def getDefault(): return NormalizerSerializer

    @staticmethod
    def _w_arr(out, t): binary.write_array(INDArray(t.reshape(1, -1) if t.dim() == 1 else t), out)

    @staticmethod
    def _r_arr(inp): return binary.read_array(inp).t.reshape(-1)

    @staticmethod
    def write(normalizer, path_or_stream):
        own = isinstance(path_or_stream, (str, bytes)) or hasattr(path_or_stream, "__fspath__")
        out = open(path_or_stream, "wb") if own else path_or_stream
        try:
            binary._write_utf(out, NormalizerSerializer.HEADER)
            out.write(struct.pack(">i", 1))
            binary._write_utf(out, normalizer.TYPE)
            W = NormalizerSerializer
            if normalizer.TYPE == "STANDARDIZE":
                out.write(struct.pack(">?", normalizer.isFitLabel()))
                W._w_arr(out, normalizer.mean_); W._w_arr(out, normalizer.std_)
                if normalizer.isFitLabel():
                    W._w_arr(out, normalizer.labelMean); W._w_arr(out, normalizer.labelStd)
            elif normalizer.TYPE == "MIN_MAX":
                out.write(struct.pack(">?dd", normalizer.isFitLabel(), normalizer.targetMin, normalizer.targetMax))
                W._w_arr(out, normalizer.min_); W._w_arr(out, normalizer.max_)
                if normalizer.isFitLabel():
                    W._w_arr(out, normalizer.labelMin); W._w_arr(out, normalizer.labelMax)
            elif normalizer.TYPE == "IMAGE_MIN_MAX":
                out.write(struct.pack(">ddd", normalizer.minRange, normalizer.maxRange, normalizer.maxPixelVal))
            elif normalizer.TYPE == "IMAGE_VGG16":
                pass
            elif normalizer.TYPE in ("MULTI_STANDARDIZE", "MULTI_MIN_MAX"):
                out.write(struct.pack(">?ii", normalizer.isFitLabel(), normalizer.numInputs(), normalizer.numOutputs() if normalizer.isFitLabel() else -1))
                if normalizer.TYPE == "MULTI_MIN_MAX":
                    a = normalizer._args
                    out.write(struct.pack(">dd", float(a[0]) if a else 0.0, float(a[1]) if len(a) > 1 else 1.0))
                for n in normalizer.inputs + (normalizer.outputs if normalizer.isFitLabel() else []):
                    if normalizer.TYPE == "MULTI_STANDARDIZE":
                        W._w_arr(out, n.mean_); W._w_arr(out, n.std_)
                    else:
                        W._w_arr(out, n.min_); W._w_arr(out, n.max_)
            else:
                raise ValueError(f"no serializer strategy for {type(normalizer).__name__}")
        finally:
            if own:
                out.close()

    @staticmethod
    def restore(path_or_stream):
        if isinstance(path_or_stream, (bytes, bytearray)):
            path_or_stream = io.BytesIO(path_or_stream)
        own = isinstance(path_or_stream, str) or hasattr(path_or_stream, "__fspath__")
        inp = open(path_or_stream, "rb") if own else path_or_stream
        try:
            R = NormalizerSerializer
            if binary._read_utf(inp) != R.HEADER:
                raise IOError("not a normalizer stream (missing NORMALIZER header)")
            (ver,) = struct.unpack(">i", inp.read(4))
            if ver != 1:
                raise IOError(f"unsupported normalizer stream version {ver}")
            typ = binary._read_utf(inp)
            if typ == "STANDARDIZE":
                (fl,) = struct.unpack(">?", inp.read(1))
                n = NormalizerStandardize(R._r_arr(inp), R._r_arr(inp))
                if fl:
                    n.labelMean, n.labelStd = R._r_arr(inp), R._r_arr(inp)
                n._fit_label = fl
                return n
            if typ == "MIN_MAX":
                fl, lo, hi = struct.unpack(">?dd", inp.read(17))
                n = NormalizerMinMaxScaler(lo, hi)
                n.min_, n.max_ = R._r_arr(inp), R._r_arr(inp)
                if fl:
                    n.labelMin, n.labelMax = R._r_arr(inp), R._r_arr(inp)
                n._fit_label = fl
                return n
            if typ == "IMAGE_MIN_MAX":
                lo, hi, mp = struct.unpack(">ddd", inp.read(24))
                n = ImagePreProcessingScaler(lo, hi)
                n.maxPixelVal = mp
                return n
            if typ == "IMAGE_VGG16":
                return VGG16ImagePreProcessor()
            if typ in ("MULTI_STANDARDIZE", "MULTI_MIN_MAX"):
                fl, ni, no = struct.unpack(">?ii", inp.read(9))
                args = ()
                if typ == "MULTI_MIN_MAX":
                    args = struct.unpack(">dd", inp.read(16))
                n = (MultiNormalizerStandardize if typ == "MULTI_STANDARDIZE" else MultiNormalizerMinMaxScaler)(*args)
                n._fit_label = fl

                def one():
                    u = n.UNDER(*args)
                    if typ == "MULTI_STANDARDIZE":
                        u.mean_, u.std_ = R._r_arr(inp), R._r_arr(inp)
                    else:
                        u.min_, u.max_ = R._r_arr(inp), R._r_arr(inp)
                    return u
                n.inputs = [one() for _ in range(ni)]
                n.outputs = [one() for _ in range(max(no, 0))] if fl else []
                return n
            raise IOError(f"unknown normalizer type {typ}")
        finally:
            if own:
                inp.close()

    read = restore
