"""Feed-forward, output, embedding and utility layers.

Parameter order and layouts follow the reference initialisers so that ``coefficients.bin`` is
interchangeable: Dense/Output ``W('f',[nIn,nOut]), b, [g]``
(``nn/params/DefaultParamInitializer.java:100-148``), Embedding same as Dense,
CenterLoss adds ``cL``, AutoEncoder adds the visible bias ``vb``
(``PretrainParamInitializer.java``), PReLU ``alpha``, ElementWiseMultiplication ``W[1,n], b``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ...ops import nnops
from ..activations import Activation, ActivationSoftmax
from ..conf.base import (BaseLayer, FeedForwardLayer, InputType, Layer, NoParamLayer, ParamSpec, RNNFormat,
                         _L, to_dropout)
from ..losses import ILossFunction, LossFunctions, LossMCXENT, LossSparseMCXENT


class DenseLayer(FeedForwardLayer):
    JAVA_CLASS = _L + "DenseLayer"
    DEFAULTS = {"hasLayerNorm": False, "hasBias": True}

    def param_specs(self):
        s = [ParamSpec("W", (self.nIn, self.nOut), "f", "weight", self.nIn, self.nOut)]
        if self.hasBias:
            s.append(ParamSpec("b", (1, self.nOut), "c", "bias", self.nIn, self.nOut))
        if self.hasLayerNorm:
            s.append(ParamSpec("g", (1, self.nOut), "c", "gain", self.nIn, self.nOut))
        return s

    def forward(self, p, x, training, mask=None, ctx=None):
        x = self.apply_dropout(x, training)
        p = self.noisy(p, training)
        if self.hasLayerNorm:
            z = nnops.linear(x, p["W"], None)
            z = nnops.layer_norm(z, p["g"].reshape(-1), p["b"].reshape(-1) if self.hasBias else None, 1e-5)
            return self.activation(z, training)
        return nnops.linear(x, p["W"], p.get("b"), self.activation, training)


class BaseOutputLayer(FeedForwardLayer):
    DEFAULTS = {"lossFunction": None, "hasBias": True}
    IS_OUTPUT = True

    def _positional(self, *args):
        if args:
            self.lossFunction = args[0]

    def _finalise(self):
        super()._finalise()
        if self.lossFunction is None:
            self.lossFunction = LossMCXENT()
        elif not isinstance(self.lossFunction, ILossFunction):
            self.lossFunction = LossFunctions.get(self.lossFunction)

    def param_specs(self):
        s = [ParamSpec("W", (self.nIn, self.nOut), "f", "weight", self.nIn, self.nOut)]
        if self.hasBias:
            s.append(ParamSpec("b", (1, self.nOut), "c", "bias", self.nIn, self.nOut))
        return s

    def pre_output(self, p, x, training):
        x = self.apply_dropout(x, training)
        p = self.noisy(p, training)
        return nnops.linear(x, p["W"], p.get("b"))

    def forward(self, p, x, training, mask=None, ctx=None):
        z = self.pre_output(p, x, training)
        if ctx is not None:
            ctx["preout"] = z
        return self.activation(z, training)

    def score_from_preout(self, preout, labels, mask=None, average=True, minibatch=None):
        lf, act = self.lossFunction, self.activation
        if preout.is_cuda and isinstance(act, ActivationSoftmax) and preout.dim() == 2 and mask is None \
                and lf.weights is None and type(lf) in (LossMCXENT, LossSparseMCXENT) and nnops.have_fused():
            s = nnops.softmax_xent(preout, labels, sparse=isinstance(lf, LossSparseMCXENT))
            return s.sum() / labels.shape[0] if average else s.sum()
        return lf.score(labels, preout, act, mask, average)

    def score_array(self, preout, labels, mask=None):
        return self.lossFunction.score_array(labels, preout, self.activation, mask)


class OutputLayer(BaseOutputLayer):
    JAVA_CLASS = _L + "OutputLayer"


class LossLayer(BaseOutputLayer):
    """Loss without parameters: activations of the previous layer are the pre-output."""
    JAVA_CLASS = _L + "LossLayer"
    HAS_PARAMS = False

    def param_specs(self):
        return []

    def setNIn(self, input_type, override):
        if input_type.kind in (InputType.FF, InputType.RNN):
            self.nIn = self.nOut = input_type.size

    def pre_output(self, p, x, training):
        return x

    def output_type(self, it):
        return it


class RnnOutputLayer(BaseOutputLayer):
    """Output layer over [mb, n, T] activations; the loss is applied per time step."""
    JAVA_CLASS = _L + "RnnOutputLayer"
    DEFAULTS = {"rnnDataFormat": RNNFormat.NCW}

    def preprocessor_for(self, input_type):
        from ..conf.preprocessors import FeedForwardToRnnPreProcessor
        if input_type.kind == InputType.FF:
            return FeedForwardToRnnPreProcessor(self.rnnDataFormat)
        return None

    def output_type(self, it):
        return InputType.recurrent(self.nOut, getattr(it, "timeSeriesLength", -1), self.rnnDataFormat)

    def _to2d(self, x, time_major=False):
        """[mb, n, T] (or [mb, T, n]) -> rows.  Row order is (example, time) unless ``time_major``: the recurrent kernels store their
        output time-major, and taking the rows in (time, example) order then needs no copy (the loss is a sum over rows)."""
        if time_major:
            x = x.permute(2, 0, 1) if self.rnnDataFormat == RNNFormat.NCW else x.permute(1, 0, 2)
        elif self.rnnDataFormat == RNNFormat.NCW:
            x = x.permute(0, 2, 1)
        return x.reshape(-1, x.shape[2])

    def _is_time_major(self, x):
        if x.dim() != 3:
            return False
        return (x.permute(2, 0, 1) if self.rnnDataFormat == RNNFormat.NCW else x.permute(1, 0, 2)).is_contiguous() and not x.is_contiguous()

    def pre_output(self, p, x, training):
        x = self.apply_dropout(x, training)
        mb = x.shape[0]
        tm = self._is_time_major(x)
        z = nnops.linear(self._to2d(x, tm), p["W"], p.get("b"))
        z._rows_time_major = tm                   # read back by forward / score_from_preout for the same row order
        return z, mb

    def forward(self, p, x, training, mask=None, ctx=None):
        z, mb = self.pre_output(p, x, training)
        if ctx is not None:
            ctx["preout"] = z
        a = self.activation(z, training)
        if getattr(z, "_rows_time_major", False):
            a = a.reshape(-1, mb, self.nOut)                                       # [T, mb, nOut]
            return a.permute(1, 2, 0) if self.rnnDataFormat == RNNFormat.NCW else a.permute(1, 0, 2)
        a = a.reshape(mb, -1, self.nOut)
        return a.permute(0, 2, 1) if self.rnnDataFormat == RNNFormat.NCW else a

    def labels2d(self, labels, time_major=False):
        if labels.dim() == 3:
            return self._to2d(labels, time_major)
        if labels.dim() == 2 and isinstance(self.lossFunction, LossSparseMCXENT):
            return (labels.t() if time_major else labels).reshape(-1, 1)
        return labels

    def score_from_preout(self, preout, labels, mask=None, average=True, minibatch=None):
        mb = minibatch or labels.shape[0]
        tm = getattr(preout, "_rows_time_major", False)
        l2 = self.labels2d(labels, tm)
        m2 = (mask.t() if tm and mask.dim() == 2 else mask).reshape(-1) if mask is not None else None
        if isinstance(self.lossFunction, LossSparseMCXENT):
            l2 = l2.reshape(-1)
        s = BaseOutputLayer.score_from_preout(self, preout, l2, m2, average=False)
        return s / mb if average else s


class RnnLossLayer(RnnOutputLayer):
    JAVA_CLASS = _L + "RnnLossLayer"
    HAS_PARAMS = False

    def param_specs(self):
        return []

    def setNIn(self, input_type, override):
        self.nIn = self.nOut = input_type.size

    def pre_output(self, p, x, training):
        return self._to2d(x), x.shape[0]


class CnnLossLayer(BaseOutputLayer):
    """Per-pixel loss over [mb, c, h, w] activations (``CnnLossLayer.java``)."""
    JAVA_CLASS = _L + "CnnLossLayer"
    HAS_PARAMS = False
    DEFAULTS = {"format": "NCHW"}

    def preprocessor_for(self, input_type):
        return None                      # consumes the convolutional activations as they are

    def param_specs(self):
        return []

    def setNIn(self, input_type, override):
        pass

    def output_type(self, it):
        return it

    def _to2d(self, x):
        if self.format == "NCHW":
            x = x.permute(0, 2, 3, 1)
        return x.reshape(-1, x.shape[-1])

    def forward(self, p, x, training, mask=None, ctx=None):
        z = self._to2d(x)
        if ctx is not None:
            ctx["preout"] = z
        a = self.activation(z, training)
        if self.format == "NCHW":
            return a.reshape(x.shape[0], x.shape[2], x.shape[3], x.shape[1]).permute(0, 3, 1, 2)
        return a.reshape(x.shape)

    def score_from_preout(self, preout, labels, mask=None, average=True, minibatch=None):
        mb = minibatch or labels.shape[0]
        s = self.lossFunction.score(self._to2d(labels), preout, self.activation,
                                    mask.reshape(-1) if mask is not None else None, average=False)
        return s / mb if average else s


class Cnn3DLossLayer(CnnLossLayer):
    JAVA_CLASS = _L + "Cnn3DLossLayer"
    DEFAULTS = {"dataFormat": "NCDHW"}

    def _to2d(self, x):
        if self.dataFormat == "NCDHW":
            x = x.permute(0, 2, 3, 4, 1)
        return x.reshape(-1, x.shape[-1])

    def forward(self, p, x, training, mask=None, ctx=None):
        z = self._to2d(x)
        if ctx is not None:
            ctx["preout"] = z
        a = self.activation(z, training)
        if self.dataFormat == "NCDHW":
            return a.reshape(x.shape[0], x.shape[2], x.shape[3], x.shape[4], x.shape[1]).permute(0, 4, 1, 2, 3)
        return a.reshape(x.shape)


class CenterLossOutputLayer(BaseOutputLayer):
    """Softmax loss + ``lambda/2 * ||f - c_y||^2`` with per-class centres updated by moving
    average rate ``alpha`` (``CenterLossOutputLayer.java``, ``CenterLossParamInitializer.java``)."""
    JAVA_CLASS = _L + "CenterLossOutputLayer"
    DEFAULTS = {"alpha": 0.05, "lambda_": 2e-4, "gradientCheck": False}

    def param_specs(self):
        s = super().param_specs()
        s.append(ParamSpec("cL", (self.nOut, self.nIn), "c", "weight", self.nIn, self.nOut, init=0.0))
        return s

    def forward(self, p, x, training, mask=None, ctx=None):
        if ctx is not None:
            ctx["center_in"] = x
            ctx["centers"] = p["cL"]
        return super().forward(p, x, training, mask, ctx)

    def extra_score(self, ctx, labels):
        x, c = ctx["center_in"], ctx["centers"]
        cy = labels.to(c.dtype) @ c
        return 0.5 * self.lambda_ * ((x - cy) ** 2).sum() / labels.shape[0]

    def to_json(self):
        d = super().to_json()
        d["lambda"] = d.pop("lambda_")
        return d


class ActivationLayer(NoParamLayer):
    JAVA_CLASS = _L + "ActivationLayer"
    DEFAULTS = {"activation": None}
    INHERIT = ("activation",)

    def _positional(self, *args):
        if args:
            self.activation = args[0]
            self._explicit.add("activation")       # a positional value must not be replaced by the global default

    def _finalise(self):
        super()._finalise()
        if self.activation is not None:
            self.activation = Activation.get(self.activation)

    def forward(self, p, x, training, mask=None, ctx=None):
        return (self.activation or Activation.get("IDENTITY"))(x, training)


class DropoutLayer(FeedForwardLayer):
    JAVA_CLASS = _L + "DropoutLayer"
    HAS_PARAMS = False

    def _positional(self, *args):
        if args:
            self.dropOut = args[0]
            self._explicit.add("dropOut")

    def param_specs(self):
        return []

    def setNIn(self, input_type, override):
        pass

    def output_type(self, it):
        return it

    def preprocessor_for(self, it):
        return None

    def forward(self, p, x, training, mask=None, ctx=None):
        return self.apply_dropout(x, training)


class EmbeddingLayer(FeedForwardLayer):
    """Index -> row lookup; input [mb,1] (or [mb]) of class indices."""
    JAVA_CLASS = _L + "EmbeddingLayer"
    DEFAULTS = {"hasBias": False}

    def param_specs(self):
        s = [ParamSpec("W", (self.nIn, self.nOut), "f", "weight", self.nIn, self.nOut)]
        if self.hasBias:
            s.append(ParamSpec("b", (1, self.nOut), "c", "bias", self.nIn, self.nOut))
        return s

    def preprocessor_for(self, it):
        return None

    def forward(self, p, x, training, mask=None, ctx=None):
        idx = x.reshape(x.shape[0]).long()
        z = p["W"][idx]
        if self.hasBias:
            z = z + p["b"]
        return self.apply_dropout(self.activation(z, training), training)


class EmbeddingSequenceLayer(FeedForwardLayer):
    """[mb, T] (or [mb,1,T]) indices -> [mb, nOut, T]."""
    JAVA_CLASS = _L + "EmbeddingSequenceLayer"
    DEFAULTS = {"hasBias": False, "inputLength": 1, "inferInputLength": True, "outputFormat": RNNFormat.NCW}

    def param_specs(self):
        s = [ParamSpec("W", (self.nIn, self.nOut), "f", "weight", self.nIn, self.nOut)]
        if self.hasBias:
            s.append(ParamSpec("b", (1, self.nOut), "c", "bias", self.nIn, self.nOut))
        return s

    def preprocessor_for(self, it):
        return None

    def output_type(self, it):
        return InputType.recurrent(self.nOut, self.inputLength, self.outputFormat)

    def forward(self, p, x, training, mask=None, ctx=None):
        if x.dim() == 3:
            x = x[:, 0, :]
        z = p["W"][x.long()]
        if self.hasBias:
            z = z + p["b"].reshape(1, 1, -1)
        z = self.activation(z, training)
        return z.permute(0, 2, 1) if self.outputFormat == RNNFormat.NCW else z


class PReLULayer(BaseLayer):
    JAVA_CLASS = _L + "PReLULayer"
    DEFAULTS = {"inputShape": None, "sharedAxes": None, "sharedAxesChannelsLast": None}
    JSON_SKIP = ("sharedAxesChannelsLast",)

    def setNIn(self, input_type, override):
        if self.inputShape is None:
            self.inputShape = input_type.getShape()
        if self.sharedAxesChannelsLast and self.sharedAxes is None:
            # axes given for a channels-last activation (the Keras convention): the last one is the channel axis, which sits first here
            n = len(self.inputShape)
            self.sharedAxes = sorted(1 if a == n else a + 1 for a in self.sharedAxesChannelsLast)

    def _alpha_shape(self):
        shp = list(self.inputShape)
        for a in (self.sharedAxes or []):
            shp[a - 1] = 1
        return tuple(shp)

    def param_specs(self):
        shp = self._alpha_shape()
        n = 1
        for s in shp:
            n *= s
        return [ParamSpec("W", shp, "c", "weight", n, n, init=0.0)]

    def forward(self, p, x, training, mask=None, ctx=None):
        a = p["W"].unsqueeze(0)
        return torch.where(x >= 0, x, x * a)


class ElementWiseMultiplicationLayer(FeedForwardLayer):
    JAVA_CLASS = _L + "misc.ElementWiseMultiplicationLayer"

    def param_specs(self):
        return [ParamSpec("W", (1, self.nOut), "c", "weight", self.nIn, self.nOut),
                ParamSpec("b", (1, self.nOut), "c", "bias", self.nIn, self.nOut)]

    def forward(self, p, x, training, mask=None, ctx=None):
        return self.activation(self.apply_dropout(x, training) * p["W"] + p["b"], training)


class RepeatVector(FeedForwardLayer):
    JAVA_CLASS = _L + "misc.RepeatVector"
    HAS_PARAMS = False
    DEFAULTS = {"n": 1, "dataFormat": RNNFormat.NCW}

    def _positional(self, *args):
        if args:
            self.n = args[0]

    def param_specs(self):
        return []

    def setNIn(self, it, override):
        self.nIn = self.nOut = it.size

    def output_type(self, it):
        return InputType.recurrent(it.size, self.n, self.dataFormat)

    def preprocessor_for(self, it):
        return None

    def forward(self, p, x, training, mask=None, ctx=None):
        y = x.unsqueeze(2).expand(-1, -1, self.n)
        return y if self.dataFormat == RNNFormat.NCW else y.permute(0, 2, 1)


class AutoEncoder(FeedForwardLayer):
    """Denoising auto-encoder (``AutoEncoder.java``): params ``W, b, vb``; unsupervised score is
    the reconstruction loss of ``decode(encode(corrupt(x)))``."""
    JAVA_CLASS = _L + "AutoEncoder"
    DEFAULTS = {"corruptionLevel": 0.3, "sparsity": 0.0, "lossFunction": None, "visibleBiasInit": 0.0}

    def _finalise(self):
        super()._finalise()
        if self.lossFunction is None:
            self.lossFunction = LossFunctions.get("MSE")
        elif not isinstance(self.lossFunction, ILossFunction):
            self.lossFunction = LossFunctions.get(self.lossFunction)

    def param_specs(self):
        return [ParamSpec("W", (self.nIn, self.nOut), "f", "weight", self.nIn, self.nOut),
                ParamSpec("b", (1, self.nOut), "c", "bias", self.nIn, self.nOut),
                ParamSpec("vb", (1, self.nIn), "c", "bias", self.nIn, self.nOut, init=self.visibleBiasInit)]

    def is_pretrain_param(self, name):
        return name == "vb"

    def encode(self, p, x, training):
        return self.activation(x @ p["W"] + p["b"], training)

    def decode(self, p, h, training):
        return self.activation(h @ p["W"].t() + p["vb"], training)

    def forward(self, p, x, training, mask=None, ctx=None):
        return self.encode(p, self.apply_dropout(x, training), training)

    def pretrain_score(self, p, x):
        xc = x
        if self.corruptionLevel > 0:
            xc = x * (torch.rand_like(x) >= self.corruptionLevel).to(x.dtype)
        recon_pre = self.encode(p, xc, True) @ p["W"].t() + p["vb"]
        return self.lossFunction.score(x, recon_pre, self.activation, None, True)


class FrozenLayer(Layer):
    """Wrapper that stops gradients to the wrapped layer's parameters (``misc/FrozenLayer.java``)."""
    JAVA_CLASS = _L + "misc.FrozenLayer"
    DEFAULTS = {"layer": None}
    FROZEN = True

    def _positional(self, *args):
        if args:
            self.layer = args[0]

    @property
    def HAS_PARAMS(self):
        return self.layer.HAS_PARAMS

    def __getattr__(self, item):
        if item in ("layer", "_explicit") or item.startswith("__"):
            raise AttributeError(item)
        return getattr(self.layer, item)

    def apply_global(self, g):
        self.layer.apply_global(g)

    def resolved(self):
        if hasattr(self.layer, "resolved"):
            self.layer.resolved()
        return self

    def setNIn(self, it, override):
        self.layer.setNIn(it, override)

    def output_type(self, it):
        return self.layer.output_type(it)

    def preprocessor_for(self, it):
        return self.layer.preprocessor_for(it)

    def param_specs(self):
        return self.layer.param_specs()

    def regularizers(self, spec):
        return []

    def updater_for(self, spec):
        from ..updaters import NoOp
        return NoOp()

    def forward(self, p, x, training, mask=None, ctx=None):
        return self.layer.forward({k: v.detach() for k, v in p.items()}, x, False, mask, ctx)

    def to_json(self):
        return {"@class": self.JAVA_CLASS, "layer": self.layer.to_json()}


class FrozenLayerWithBackprop(FrozenLayer):
    """Frozen parameters, but epsilons still flow to earlier layers."""
    JAVA_CLASS = _L + "misc.FrozenLayerWithBackprop"

    def forward(self, p, x, training, mask=None, ctx=None):
        return self.layer.forward({k: v.detach() for k, v in p.items()}, x, training, mask, ctx)


class MaskLayer(NoParamLayer):
    """Zeroes activations at masked time steps / examples (``util/MaskLayer.java``)."""
    JAVA_CLASS = _L + "util.MaskLayer"

    def forward(self, p, x, training, mask=None, ctx=None):
        if mask is None:
            return x
        m = mask
        if x.dim() == 3:
            m = mask.unsqueeze(1)
        elif x.dim() == 2 and mask.dim() == 1:
            m = mask.unsqueeze(1)
        elif x.dim() == 4:
            m = mask.reshape(mask.shape[0], 1, 1, 1) if mask.dim() <= 2 else mask
        return x * m.to(x.dtype)


class MaskZeroLayer(Layer):
    """Wraps a recurrent layer; time steps whose input equals ``maskingValue`` are masked."""
    JAVA_CLASS = _L + "util.MaskZeroLayer"
    DEFAULTS = {"underlying": None, "maskingValue": 0.0}

    @property
    def HAS_PARAMS(self):
        return self.underlying.HAS_PARAMS

    def apply_global(self, g): self.underlying.apply_global(g)
    def resolved(self):
        self.underlying.resolved(); return self
    def setNIn(self, it, o): self.underlying.setNIn(it, o)
    def output_type(self, it): return self.underlying.output_type(it)
    def preprocessor_for(self, it): return self.underlying.preprocessor_for(it)
    def param_specs(self): return self.underlying.param_specs()
    def regularizers(self, s): return self.underlying.regularizers(s)
    def updater_for(self, s): return self.underlying.updater_for(s)

    def forward(self, p, x, training, mask=None, ctx=None):
        m = (x != self.maskingValue).any(dim=1).to(x.dtype)   # [mb, T]
        return self.underlying.forward(p, x, training, m, ctx)

    def to_json(self):
        return {"@class": self.JAVA_CLASS, "maskingValue": self.maskingValue, "underlying": self.underlying.to_json()}
