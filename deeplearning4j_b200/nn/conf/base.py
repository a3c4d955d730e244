"""Configuration primitives shared by every layer: ``InputType``, enums, dropout, constraints,
weight noise and the ``Layer`` base class with its fluent ``Builder``.

Reference shapes: ``deeplearning4j-nn/.../nn/conf/inputs/InputType.java``,
``nn/conf/layers/Layer.java:51-69``, ``BaseLayer.java:52-62``, ``FeedForwardLayer.java:39-41``,
``nn/conf/dropout/*.java``, ``nn/conf/constraint/*.java``.

A layer object here is both the DL4J *configuration* (JSON-serialisable, ``@class`` typed) and
the *runtime*: ``param_specs`` describes its slice of the flattened parameter buffer in DL4J's
order and ``forward`` is a differentiable torch function over views of that buffer, so the
network keeps one flat params / gradients / updater-state triple exactly like
``MultiLayerNetwork.flattenedParams``.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Any, Optional

import torch
import torch.nn.functional as F

from ..activations import Activation, IActivation
from ..updaters import (IUpdater, L1Regularization, L2Regularization, Regularization, WeightDecay,
                        regularization_from_json, updater_from_json)
from ..weights import IWeightInit, WeightInit, Distribution

_L = "org.deeplearning4j.nn.conf.layers."


# --------------------------------------------------------------------------- enums
class ConvolutionMode:
    Strict = "Strict"; Truncate = "Truncate"; Same = "Same"; Causal = "Causal"


class PoolingType:
    MAX = "MAX"; AVG = "AVG"; SUM = "SUM"; PNORM = "PNORM"


class CNN2DFormat:
    NCHW = "NCHW"; NHWC = "NHWC"


class RNNFormat:
    NCW = "NCW"; NWC = "NWC"


class BackpropType:
    Standard = "Standard"; TruncatedBPTT = "TruncatedBPTT"


class WorkspaceMode:
    ENABLED = "ENABLED"; NONE = "NONE"


class CacheMode:
    NONE = "NONE"; HOST = "HOST"; DEVICE = "DEVICE"


class OptimizationAlgorithm:
    STOCHASTIC_GRADIENT_DESCENT = "STOCHASTIC_GRADIENT_DESCENT"


class GradientNormalization:
    None_ = "None"; RenormalizeL2PerLayer = "RenormalizeL2PerLayer"
    RenormalizeL2PerParamType = "RenormalizeL2PerParamType"
    ClipElementWiseAbsoluteValue = "ClipElementWiseAbsoluteValue"
    ClipL2PerLayer = "ClipL2PerLayer"; ClipL2PerParamType = "ClipL2PerParamType"


# --------------------------------------------------------------------------- InputType
class InputType:
    FF = "FeedForward"; RNN = "Recurrent"; CNN = "Convolutional"; CNNFlat = "ConvolutionalFlat"; CNN3D = "Convolutional3D"

    def __init__(self, kind, **kw):
        self.kind = kind
        self.__dict__.update(kw)

    @staticmethod
    def feedForward(size, timeDistributedFormat=None):
        return InputType(InputType.FF, size=int(size))

    @staticmethod
    def recurrent(size, timeSeriesLength=-1, format=RNNFormat.NCW):
        return InputType(InputType.RNN, size=int(size), timeSeriesLength=int(timeSeriesLength), format=format)

    @staticmethod
    def convolutional(height, width, channels, format=CNN2DFormat.NCHW):
        return InputType(InputType.CNN, height=int(height), width=int(width), channels=int(channels), format=format)

    @staticmethod
    def convolutionalFlat(height, width, channels):
        return InputType(InputType.CNNFlat, height=int(height), width=int(width), channels=int(channels))

    @staticmethod
    def convolutional3D(depth, height, width, channels, dataFormat="NCDHW"):
        return InputType(InputType.CNN3D, depth=int(depth), height=int(height), width=int(width),
                         channels=int(channels), dataFormat=dataFormat)

    def arrayElementsPerExample(self):
        if self.kind == InputType.FF:
            return self.size
        if self.kind == InputType.RNN:
            return self.size * max(self.timeSeriesLength, 1)
        if self.kind == InputType.CNN3D:
            return self.depth * self.height * self.width * self.channels
        return self.height * self.width * self.channels

    def getShape(self, includeBatch=False):
        if self.kind == InputType.FF:
            s = [self.size]
        elif self.kind == InputType.RNN:
            s = [self.size, self.timeSeriesLength] if self.format == RNNFormat.NCW else [self.timeSeriesLength, self.size]
        elif self.kind == InputType.CNN:
            s = [self.channels, self.height, self.width] if self.format == CNN2DFormat.NCHW else [self.height, self.width, self.channels]
        elif self.kind == InputType.CNNFlat:
            s = [self.height * self.width * self.channels]
        else:
            s = [self.channels, self.depth, self.height, self.width]
        return ([-1] if includeBatch else []) + s

    def to_json(self):
        d = {"@class": "org.deeplearning4j.nn.conf.inputs.InputType$InputType" + self.kind}
        d.update({k: v for k, v in self.__dict__.items() if k != "kind"})
        return d

    @staticmethod
    def from_json(d):
        if d is None:
            return None
        kind = d["@class"].rsplit("InputType", 1)[-1]
        return InputType(kind, **{k: v for k, v in d.items() if k != "@class"})

    def __eq__(self, o):
        return isinstance(o, InputType) and self.__dict__ == o.__dict__

    def __repr__(self):
        return "InputType" + self.kind + "(" + ", ".join(f"{k}={v}" for k, v in self.__dict__.items() if k != "kind") + ")"


# --------------------------------------------------------------------------- dropout
_D = "org.deeplearning4j.nn.conf.dropout."


class IDropout:
    JAVA = ""; FIELDS: tuple = ()
    def apply(self, x, training, iteration=0, epoch=0): raise NotImplementedError
    def to_json(self):
        d = {"@class": _D + self.JAVA}
        for f in self.FIELDS:
            d[f] = getattr(self, f)
        return d
    def __eq__(self, o): return type(self) is type(o) and self.to_json() == o.to_json()
    def __hash__(self): return hash(type(self))


class Dropout(IDropout):
    """Inverted dropout; ``p`` is the *retain* probability, as in DL4J."""
    JAVA = "Dropout"; FIELDS = ("p",)
    def __init__(self, p=0.5): self.p = float(p)
    def apply(self, x, training, iteration=0, epoch=0):
        if not training or self.p >= 1.0:
            return x
        return F.dropout(x, 1.0 - self.p, True)


class SpatialDropout(Dropout):
    JAVA = "SpatialDropout"
    def apply(self, x, training, iteration=0, epoch=0):
        if not training or self.p >= 1.0:
            return x
        shape = list(x.shape[:2]) + [1] * (x.dim() - 2)
        mask = (torch.rand(shape, device=x.device) < self.p).to(x.dtype) / self.p
        return x * mask


class AlphaDropout(Dropout):
    JAVA = "AlphaDropout"
    def apply(self, x, training, iteration=0, epoch=0):
        return F.alpha_dropout(x, 1.0 - self.p, training)


class GaussianDropout(IDropout):
    JAVA = "GaussianDropout"; FIELDS = ("rate",)
    def __init__(self, rate=0.5): self.rate = float(rate)
    def apply(self, x, training, iteration=0, epoch=0):
        if not training:
            return x
        std = math.sqrt(self.rate / (1.0 - self.rate))
        return x * (1.0 + std * torch.randn_like(x))


class GaussianNoise(IDropout):
    JAVA = "GaussianNoise"; FIELDS = ("stddev",)
    def __init__(self, stddev=0.1): self.stddev = float(stddev)
    def apply(self, x, training, iteration=0, epoch=0):
        return x + self.stddev * torch.randn_like(x) if training else x


DROPOUTS = {c.JAVA: c for c in (Dropout, SpatialDropout, AlphaDropout, GaussianDropout, GaussianNoise)}


def dropout_from_json(d):
    if d is None:
        return None
    cls = DROPOUTS[d["@class"].rsplit(".", 1)[-1]]
    return cls(**{k: v for k, v in d.items() if k in cls.FIELDS})


def to_dropout(v):
    if v is None or isinstance(v, IDropout):
        return v
    v = float(v)
    return None if v == 0.0 or v >= 1.0 else Dropout(v)


# --------------------------------------------------------------------------- constraints
_C = "org.deeplearning4j.nn.conf.constraint."


class LayerConstraint:
    JAVA = ""; FIELDS: tuple = ()
    def __init__(self, dims=(1,)): self.dimensions = list(dims); self.params = None
    def apply(self, w): raise NotImplementedError
    def to_json(self):
        d = {"@class": _C + self.JAVA, "dimensions": self.dimensions, "params": sorted(self.params) if self.params else None}
        for f in self.FIELDS:
            d[f] = getattr(self, f)
        return d
    def _norm(self, w):
        dims = [d for d in self.dimensions if d < w.dim()]
        return w.norm(2, dim=dims, keepdim=True) if dims else w.norm(2)


class MaxNormConstraint(LayerConstraint):
    JAVA = "MaxNormConstraint"; FIELDS = ("maxNorm",)
    def __init__(self, maxNorm=1.0, *dims):
        super().__init__(dims or (1,)); self.maxNorm = float(maxNorm)
    def apply(self, w):
        n = self._norm(w)
        w.mul_(torch.clamp(n, max=self.maxNorm) / (n + 1e-8))


class MinMaxNormConstraint(LayerConstraint):
    JAVA = "MinMaxNormConstraint"; FIELDS = ("min", "max", "rate")
    def __init__(self, min=0.0, max=1.0, rate=1.0, *dims):
        super().__init__(dims or (1,)); self.min, self.max, self.rate = float(min), float(max), float(rate)
    def apply(self, w):
        n = self._norm(w)
        target = self.rate * torch.clamp(n, self.min, self.max) + (1 - self.rate) * n
        w.mul_(target / (n + 1e-8))


class NonNegativeConstraint(LayerConstraint):
    JAVA = "NonNegativeConstraint"
    def apply(self, w): w.clamp_(min=0.0)


class UnitNormConstraint(LayerConstraint):
    JAVA = "UnitNormConstraint"
    def __init__(self, *dims): super().__init__(dims or (1,))
    def apply(self, w): w.div_(self._norm(w) + 1e-8)


CONSTRAINTS = {c.JAVA: c for c in (MaxNormConstraint, MinMaxNormConstraint, NonNegativeConstraint, UnitNormConstraint)}


def constraint_from_json(d):
    cls = CONSTRAINTS[d["@class"].rsplit(".", 1)[-1]]
    o = cls.__new__(cls)
    o.dimensions = d.get("dimensions") or [1]
    o.params = set(d["params"]) if d.get("params") else None
    for f in cls.FIELDS:
        setattr(o, f, d.get(f))
    return o


# --------------------------------------------------------------------------- weight noise
_WN = "org.deeplearning4j.nn.conf.weightnoise."


class DropConnect:
    """Drops individual weights at training time (``weightnoise/DropConnect.java``)."""
    def __init__(self, weightRetainProb=0.5, applyToBiases=False):
        self.weightRetainProb, self.applyToBiases = float(weightRetainProb), applyToBiases
    def apply(self, name, is_bias, w, training):
        if not training or (is_bias and not self.applyToBiases):
            return w
        return F.dropout(w, 1.0 - self.weightRetainProb, True)
    def to_json(self):
        return {"@class": _WN + "DropConnect", "applyToBiases": self.applyToBiases, "weightRetainProb": self.weightRetainProb}


class WeightNoise:
    """Additive or multiplicative noise on weights (``weightnoise/WeightNoise.java``)."""
    def __init__(self, distribution: Distribution, applyToBias=False, additive=True):
        self.distribution, self.applyToBias, self.additive = distribution, applyToBias, additive
    def apply(self, name, is_bias, w, training):
        if not training or (is_bias and not self.applyToBias):
            return w
        noise = torch.empty_like(w)
        self.distribution.sample_(noise, None)
        return w + noise if self.additive else w * noise
    def to_json(self):
        return {"@class": _WN + "WeightNoise", "additive": self.additive, "applyToBias": self.applyToBias,
                "distribution": self.distribution.to_json()}


def weight_noise_from_json(d):
    if d is None:
        return None
    from ..weights import distribution_from_json
    if d["@class"].endswith("DropConnect"):
        return DropConnect(d.get("weightRetainProb", 0.5), d.get("applyToBiases", False))
    return WeightNoise(distribution_from_json(d["distribution"]), d.get("applyToBias", False), d.get("additive", True))


# --------------------------------------------------------------------------- parameter spec
@dataclass
class ParamSpec:
    name: str
    shape: tuple            # logical shape
    order: str = "c"        # 'c' or 'f' layout inside the flat buffer
    kind: str = "weight"    # weight | bias | gain | state(no gradient-based update, e.g. BN mean/var)
    fanIn: float = 1.0
    fanOut: float = 1.0
    init: Any = None        # None -> layer's weightInitFn / biasInit by kind; float -> constant; callable(out, gen)

    @property
    def numel(self):
        n = 1
        for s in self.shape:
            n *= int(s)
        return n

    @property
    def is_bias(self):
        return self.kind == "bias"


def flat_view(flat: torch.Tensor, offset: int, spec: ParamSpec) -> torch.Tensor:
    """Logical-shape view of ``spec`` inside ``flat`` honouring its 'c' / 'f' layout."""
    seg = flat[offset:offset + spec.numel]
    if spec.order == "f" and len(spec.shape) > 1:
        nd = len(spec.shape)
        return seg.view(tuple(reversed(spec.shape))).permute(*reversed(range(nd)))
    return seg.view(spec.shape)


# --------------------------------------------------------------------------- builder
class _Builder:
    """Fluent builder: ``DenseLayer.Builder().nIn(4).nOut(3).activation("relu").build()``.

    Every configuration field doubles as a setter method; a few DL4J conveniences (``l1``,
    ``l2``, ``weightDecay``, ``dropOut``, ``dist``, ``updater``, ``name``) are translated.
    """

    def __init__(self, cls, *args, **kw):
        self._cls, self._args, self._kw = cls, args, dict(kw)

    def __getattr__(self, item):
        if item.startswith("_"):
            raise AttributeError(item)

        def setter(*v):
            self._kw[item] = v[0] if len(v) == 1 else tuple(v)
            return self
        return setter

    def build(self):
        return self._cls(*self._args, **self._kw)


_ALIASES = {"name": "layerName", "activationFn": "activation", "weightInitFn": "weightInit", "iUpdater": "updater",
            "iDropout": "dropOut", "lossFn": "lossFunction", "convolutionType": "convolutionMode"}


class Layer:
    """Base of all layer configs (``nn/conf/layers/Layer.java``)."""
    JAVA_CLASS = _L + "Layer"
    # field -> default; subclasses extend through DEFAULTS (merged along the MRO)
    DEFAULTS: dict = {"layerName": None, "dropOut": None, "constraints": None}
    # fields inherited from the global NeuralNetConfiguration.Builder when left unset
    INHERIT: tuple = ("dropOut",)
    HAS_PARAMS = False

    def __init__(self, *args, **kw):
        merged = {}
        for c in reversed(type(self).__mro__):
            merged.update(getattr(c, "DEFAULTS", {}))
        self._explicit = set()
        for k, v in merged.items():
            setattr(self, k, copy.copy(v) if isinstance(v, (list, dict)) else v)
        self._positional(*args)
        for k, v in kw.items():
            k = _ALIASES.get(k, k)
            self._set(k, v)
        self._finalise()

    # -- construction helpers
    def _positional(self, *args):
        if args:
            raise TypeError(f"{type(self).__name__} takes keyword arguments only")

    def _set(self, k, v):
        if k == "l1":
            self._add_reg(L1Regularization(v), False); return
        if k == "l2":
            self._add_reg(L2Regularization(v), False); return
        if k == "l1Bias":
            self._add_reg(L1Regularization(v), True); return
        if k == "l2Bias":
            self._add_reg(L2Regularization(v), True); return
        if k == "weightDecay":
            self._add_reg(WeightDecay(*(v if isinstance(v, tuple) else (v,))), False); return
        if k == "weightDecayBias":
            self._add_reg(WeightDecay(*(v if isinstance(v, tuple) else (v,))), True); return
        if k == "dist":
            self.weightInit = WeightInit.get(v); self._explicit.add("weightInit"); return
        if not hasattr(self, k):
            raise TypeError(f"{type(self).__name__} has no configuration field '{k}'")
        setattr(self, k, v)
        self._explicit.add(k)

    def _add_reg(self, reg, bias):
        key = "regularizationBias" if bias else "regularization"
        cur = list(getattr(self, key, None) or [])
        cur = [r for r in cur if type(r) is not type(reg)]
        if reg.value(0, 0) != 0 if not hasattr(reg.coeff, "valueAt") else True:
            cur.append(reg)
        setattr(self, key, cur)
        self._explicit.add(key)

    def _finalise(self):
        self.dropOut = to_dropout(self.dropOut)

    @classmethod
    def Builder(cls, *args, **kw):
        return _Builder(cls, *args, **kw)

    @classmethod
    def builder(cls, *args, **kw):
        return _Builder(cls, *args, **kw)

    # -- global-default inheritance (NeuralNetConfiguration.Builder -> layer)
    def apply_global(self, g: dict):
        for f in self._inherit_fields():
            if f not in self._explicit and f in g and g[f] is not None and hasattr(self, f):
                v = g[f]
                setattr(self, f, copy.deepcopy(v) if not isinstance(v, (str, int, float, bool)) else v)
        self._finalise()

    def _inherit_fields(self):
        out = []
        for c in type(self).__mro__:
            out.extend(getattr(c, "INHERIT", ()))
        return out

    # -- shape inference / params
    def setNIn(self, input_type: InputType, override: bool):
        pass

    def output_type(self, input_type: InputType) -> InputType:
        return input_type

    def param_specs(self) -> list:
        return []

    def num_params(self):
        return sum(s.numel for s in self.param_specs())

    def preprocessor_for(self, input_type: InputType):
        return None

    def is_pretrain_param(self, name):
        return False

    # -- runtime
    def forward(self, p: dict, x, training: bool, mask=None, ctx=None):
        raise NotImplementedError(type(self).__name__)

    def feed_forward_mask(self, mask, input_type=None):
        return mask

    def apply_dropout(self, x, training):
        return self.dropOut.apply(x, training) if self.dropOut is not None else x

    def regularizers(self, spec: ParamSpec):
        return []

    def updater_for(self, spec: ParamSpec):
        return None

    # -- JSON
    JSON_SKIP = ()

    def to_json(self):
        d = {"@class": self.JAVA_CLASS}
        for c in reversed(type(self).__mro__):
            for k in getattr(c, "DEFAULTS", {}):
                if k in self.JSON_SKIP:
                    continue
                d[_JSON_NAMES.get(k, k)] = _to_json_value(getattr(self, k))
        return d

    @classmethod
    def from_json(cls, d):
        obj = cls.__new__(cls)
        merged = {}
        for c in reversed(cls.__mro__):
            merged.update(getattr(c, "DEFAULTS", {}))
        obj._explicit = set(merged)
        inv = {v: k for k, v in _JSON_NAMES.items()}
        for k, v in merged.items():
            setattr(obj, k, copy.copy(v) if isinstance(v, (list, dict)) else v)
        for jk, v in d.items():
            if jk == "@class":
                continue
            k = inv.get(jk, jk)
            if k in merged:
                setattr(obj, k, _from_json_value(k, v))
        obj._post_json()
        return obj

    def _post_json(self):
        pass

    def clone(self):
        return copy.deepcopy(self)

    def __repr__(self):
        return f"{type(self).__name__}({self.layerName or ''})"


_JSON_NAMES = {"activation": "activationFn", "weightInit": "weightInitFn", "updater": "iUpdater", "dropOut": "iDropout",
               "lossFunction": "lossFn", "weightInitRecurrent": "weightInitFnRecurrent"}


def _to_json_value(v):
    if hasattr(v, "to_json"):
        return v.to_json()
    if isinstance(v, (list, tuple)):
        return [_to_json_value(e) for e in v]
    if isinstance(v, dict):
        return {str(k): _to_json_value(e) for k, e in v.items()}
    return v


def _from_json_value(k, v):
    from ..losses import LossFunctions
    from ..weights import distribution_from_json
    if v is None:
        return None
    if k in ("activation", "gateActivationFn", "activationFn"):
        return Activation.from_json(v)
    if k in ("weightInit", "weightInitRecurrent"):
        return WeightInit.from_json(v)
    if k in ("updater", "biasUpdater"):
        return updater_from_json(v)
    if k == "dropOut":
        return dropout_from_json(v)
    if k == "lossFunction":
        return LossFunctions.from_json(v)
    if k in ("regularization", "regularizationBias"):
        return [regularization_from_json(e) for e in v]
    if k == "constraints":
        return [constraint_from_json(e) for e in v]
    if k == "weightNoise":
        return weight_noise_from_json(v)
    if isinstance(v, dict) and "@class" in v:
        from .registry import object_from_json
        return object_from_json(v)
    if isinstance(v, list) and v and isinstance(v[0], dict) and "@class" in v[0]:
        from .registry import object_from_json
        return [object_from_json(e) for e in v]
    return v


class BaseLayer(Layer):
    """Layers with trainable parameters (``nn/conf/layers/BaseLayer.java:52-62``)."""
    DEFAULTS = {"activation": None, "weightInit": None, "biasInit": None, "gainInit": None,
                "regularization": None, "regularizationBias": None, "updater": None, "biasUpdater": None,
                "weightNoise": None, "gradientNormalization": None, "gradientNormalizationThreshold": None}
    INHERIT = ("activation", "weightInit", "biasInit", "gainInit", "regularization", "regularizationBias", "updater",
               "biasUpdater", "weightNoise", "gradientNormalization", "gradientNormalizationThreshold")
    HAS_PARAMS = True

    def _finalise(self):
        super()._finalise()
        if self.activation is not None and not isinstance(self.activation, IActivation):
            self.activation = Activation.get(self.activation)
        if self.weightInit is not None and not isinstance(self.weightInit, IWeightInit):
            self.weightInit = WeightInit.get(self.weightInit)

    def resolved(self):
        """Fill still-missing fields with DL4J's global defaults (sigmoid, Xavier, Sgd)."""
        from ..updaters import Sgd
        if self.activation is None:
            self.activation = Activation.get("SIGMOID")
        if self.weightInit is None:
            self.weightInit = WeightInit.get("XAVIER")
        if self.biasInit is None:
            self.biasInit = 0.0
        if self.gainInit is None:
            self.gainInit = 1.0
        if self.updater is None:
            self.updater = Sgd()
        if self.gradientNormalization is None:
            self.gradientNormalization = GradientNormalization.None_
        if self.gradientNormalizationThreshold is None:
            self.gradientNormalizationThreshold = 1.0
        self.regularization = list(self.regularization or [])
        self.regularizationBias = list(self.regularizationBias or [])
        return self

    def regularizers(self, spec):
        if spec.kind == "state":
            return []
        return (self.regularizationBias if spec.is_bias else self.regularization) or []

    def updater_for(self, spec):
        if spec.kind == "state":
            from ..updaters import NoOp
            return NoOp()
        if spec.is_bias and self.biasUpdater is not None:
            return self.biasUpdater
        return self.updater

    def noisy(self, p: dict, training: bool):
        if self.weightNoise is None or not training:
            return p
        kinds = {s.name: s.is_bias for s in self.param_specs()}
        return {k: self.weightNoise.apply(k, kinds.get(k, False), v, training) for k, v in p.items()}


class FeedForwardLayer(BaseLayer):
    DEFAULTS = {"nIn": 0, "nOut": 0, "timeDistributedFormat": None}

    def setNIn(self, input_type, override):
        if self.nIn and not override:
            return
        if input_type.kind in (InputType.FF, InputType.RNN):
            self.nIn = input_type.size
        elif input_type.kind == InputType.CNN3D:
            self.nIn = input_type.arrayElementsPerExample()
        else:
            self.nIn = input_type.height * input_type.width * input_type.channels

    def output_type(self, input_type):
        if input_type is not None and input_type.kind == InputType.RNN:
            return InputType.recurrent(self.nOut, input_type.timeSeriesLength, input_type.format)
        return InputType.feedForward(self.nOut)

    def preprocessor_for(self, input_type):
        from .preprocessors import CnnToFeedForwardPreProcessor, RnnToFeedForwardPreProcessor, Cnn3DToFeedForwardPreProcessor
        if input_type.kind == InputType.CNN:
            return CnnToFeedForwardPreProcessor(input_type.height, input_type.width, input_type.channels, input_type.format)
        if input_type.kind == InputType.CNN3D:
            return Cnn3DToFeedForwardPreProcessor(input_type.depth, input_type.height, input_type.width, input_type.channels)
        if input_type.kind == InputType.RNN:
            return RnnToFeedForwardPreProcessor(input_type.format)
        return None


class NoParamLayer(Layer):
    HAS_PARAMS = False
