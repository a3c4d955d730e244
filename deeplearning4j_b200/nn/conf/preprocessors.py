"""Input pre-processors (``deeplearning4j-nn/.../nn/conf/preprocessor/*.java``): reshape
activations between feed-forward [mb,n], recurrent [mb,n,T] (NCW) and convolutional
[mb,c,h,w] layouts.  Backward passes come from autograd."""
from __future__ import annotations

import torch

from .base import InputType, CNN2DFormat, RNNFormat

_P = "org.deeplearning4j.nn.conf.preprocessor."


class InputPreProcessor:
    JAVA = ""; FIELDS: tuple = ()

    def preProcess(self, x, minibatch=None, ctx=None):
        raise NotImplementedError

    def output_type(self, it):
        return it

    def feed_forward_mask(self, mask, minibatch=None):
        return mask

    def to_json(self):
        d = {"@class": _P + self.JAVA}
        for f in self.FIELDS:
            d[f] = getattr(self, f)
        return d

    def __eq__(self, o):
        return type(self) is type(o) and self.to_json() == o.to_json()


class CnnToFeedForwardPreProcessor(InputPreProcessor):
    JAVA = "CnnToFeedForwardPreProcessor"; FIELDS = ("inputHeight", "inputWidth", "numChannels", "format")
    def __init__(self, inputHeight=0, inputWidth=0, numChannels=0, format=CNN2DFormat.NCHW):
        self.inputHeight, self.inputWidth, self.numChannels, self.format = inputHeight, inputWidth, numChannels, format
    def preProcess(self, x, minibatch=None, ctx=None):
        return x.reshape(x.shape[0], -1)
    def output_type(self, it):
        return InputType.feedForward(it.height * it.width * it.channels)


class FeedForwardToCnnPreProcessor(InputPreProcessor):
    JAVA = "FeedForwardToCnnPreProcessor"; FIELDS = ("inputHeight", "inputWidth", "numChannels")
    def __init__(self, inputHeight, inputWidth, numChannels=1):
        self.inputHeight, self.inputWidth, self.numChannels = inputHeight, inputWidth, numChannels
    def preProcess(self, x, minibatch=None, ctx=None):
        if x.dim() == 4:
            return x
        return x.reshape(x.shape[0], self.numChannels, self.inputHeight, self.inputWidth)
    def output_type(self, it):
        return InputType.convolutional(self.inputHeight, self.inputWidth, self.numChannels)


class Cnn3DToFeedForwardPreProcessor(InputPreProcessor):
    JAVA = "Cnn3DToFeedForwardPreProcessor"; FIELDS = ("inputDepth", "inputHeight", "inputWidth", "numChannels", "isNCDHW")
    def __init__(self, inputDepth=0, inputHeight=0, inputWidth=0, numChannels=0, isNCDHW=True):
        self.inputDepth, self.inputHeight, self.inputWidth, self.numChannels, self.isNCDHW = inputDepth, inputHeight, inputWidth, numChannels, isNCDHW
    def preProcess(self, x, minibatch=None, ctx=None):
        return x.reshape(x.shape[0], -1)
    def output_type(self, it):
        return InputType.feedForward(it.arrayElementsPerExample())


class FeedForwardToCnn3DPreProcessor(InputPreProcessor):
    JAVA = "FeedForwardToCnn3DPreProcessor"; FIELDS = ("inputDepth", "inputHeight", "inputWidth", "numChannels", "isNCDHW")
    def __init__(self, inputDepth, inputHeight, inputWidth, numChannels=1, isNCDHW=True):
        self.inputDepth, self.inputHeight, self.inputWidth, self.numChannels, self.isNCDHW = inputDepth, inputHeight, inputWidth, numChannels, isNCDHW
    def preProcess(self, x, minibatch=None, ctx=None):
        return x.reshape(x.shape[0], self.numChannels, self.inputDepth, self.inputHeight, self.inputWidth)
    def output_type(self, it):
        return InputType.convolutional3D(self.inputDepth, self.inputHeight, self.inputWidth, self.numChannels)


class RnnToFeedForwardPreProcessor(InputPreProcessor):
    """[mb, n, T] -> [mb*T, n] (time-major within each example, as the reference does)."""
    JAVA = "RnnToFeedForwardPreProcessor"; FIELDS = ("rnnDataFormat",)
    def __init__(self, rnnDataFormat=RNNFormat.NCW):
        self.rnnDataFormat = rnnDataFormat or RNNFormat.NCW
    def preProcess(self, x, minibatch=None, ctx=None):
        if x.dim() == 2:
            return x
        if self.rnnDataFormat == RNNFormat.NCW:
            x = x.permute(0, 2, 1)
        if ctx is not None:
            ctx["rnn_T"] = x.shape[1]
        return x.reshape(-1, x.shape[2])
    def output_type(self, it):
        return InputType.feedForward(it.size)
    def feed_forward_mask(self, mask, minibatch=None):
        return None if mask is None else mask.reshape(-1, 1) if mask.dim() == 2 else mask


class FeedForwardToRnnPreProcessor(InputPreProcessor):
    JAVA = "FeedForwardToRnnPreProcessor"; FIELDS = ("rnnDataFormat",)
    def __init__(self, rnnDataFormat=RNNFormat.NCW):
        self.rnnDataFormat = rnnDataFormat or RNNFormat.NCW
    def preProcess(self, x, minibatch=None, ctx=None):
        if x.dim() == 3:
            return x
        mb = minibatch or (ctx or {}).get("minibatch") or x.shape[0]
        x = x.reshape(mb, -1, x.shape[1])
        return x.permute(0, 2, 1) if self.rnnDataFormat == RNNFormat.NCW else x
    def output_type(self, it):
        return InputType.recurrent(it.size, -1, self.rnnDataFormat)
    def feed_forward_mask(self, mask, minibatch=None):
        return None if mask is None else mask.reshape(minibatch, -1) if minibatch else mask


class CnnToRnnPreProcessor(InputPreProcessor):
    """[mb*T, c, h, w] -> [mb, c*h*w, T]."""
    JAVA = "CnnToRnnPreProcessor"; FIELDS = ("inputHeight", "inputWidth", "numChannels", "rnnDataFormat")
    def __init__(self, inputHeight, inputWidth, numChannels, rnnDataFormat=RNNFormat.NCW):
        self.inputHeight, self.inputWidth, self.numChannels, self.rnnDataFormat = inputHeight, inputWidth, numChannels, rnnDataFormat
    def preProcess(self, x, minibatch=None, ctx=None):
        mb = minibatch or (ctx or {}).get("minibatch") or x.shape[0]
        x = x.reshape(mb, -1, self.numChannels * self.inputHeight * self.inputWidth)
        return x.permute(0, 2, 1) if self.rnnDataFormat == RNNFormat.NCW else x
    def output_type(self, it):
        return InputType.recurrent(it.height * it.width * it.channels, -1, self.rnnDataFormat)


class RnnToCnnPreProcessor(InputPreProcessor):
    """[mb, c*h*w, T] -> [mb*T, c, h, w]."""
    JAVA = "RnnToCnnPreProcessor"; FIELDS = ("inputHeight", "inputWidth", "numChannels", "rnnDataFormat")
    def __init__(self, inputHeight, inputWidth, numChannels, rnnDataFormat=RNNFormat.NCW):
        self.inputHeight, self.inputWidth, self.numChannels, self.rnnDataFormat = inputHeight, inputWidth, numChannels, rnnDataFormat
    def preProcess(self, x, minibatch=None, ctx=None):
        if self.rnnDataFormat == RNNFormat.NCW:
            x = x.permute(0, 2, 1)
        return x.reshape(-1, self.numChannels, self.inputHeight, self.inputWidth)
    def output_type(self, it):
        return InputType.convolutional(self.inputHeight, self.inputWidth, self.numChannels)


class ComposableInputPreProcessor(InputPreProcessor):
    JAVA = "ComposableInputPreProcessor"
    def __init__(self, *pps):
        self.inputPreProcessors = list(pps[0]) if len(pps) == 1 and isinstance(pps[0], (list, tuple)) else list(pps)
    def preProcess(self, x, minibatch=None, ctx=None):
        for p in self.inputPreProcessors:
            x = p.preProcess(x, minibatch, ctx)
        return x
    def output_type(self, it):
        for p in self.inputPreProcessors:
            it = p.output_type(it)
        return it
    def to_json(self):
        return {"@class": _P + self.JAVA, "inputPreProcessors": [p.to_json() for p in self.inputPreProcessors]}


def _to_channels_last(x):
    return x.permute(0, *range(2, x.dim()), 1) if x.dim() > 2 else x


def _to_channels_first(x):
    return x.permute(0, x.dim() - 1, *range(1, x.dim() - 1)) if x.dim() > 2 else x


def _type_of_channels_last(shape):
    """InputType of an activation whose Keras (channels-last, no batch axis) shape is ``shape``."""
    s = [int(v) for v in shape]
    if len(s) == 1:
        return InputType.feedForward(s[0])
    if len(s) == 2:
        return InputType.recurrent(s[1], s[0])
    if len(s) == 3:
        return InputType.convolutional(s[0], s[1], s[2])
    if len(s) == 4:
        return InputType.convolutional3D(s[0], s[1], s[2], s[3])
    raise ValueError(f"no input type for a rank-{len(s) + 1} activation")


def _channels_last_shape(it):
    if it.kind == InputType.CNN:
        return [it.height, it.width, it.channels]
    if it.kind == InputType.RNN:
        return [it.timeSeriesLength, it.size]
    if it.kind == InputType.CNN3D:
        return [it.depth, it.height, it.width, it.channels]
    return [it.size]


class ReshapePreprocessor(InputPreProcessor):
    """Keras ``Reshape`` (``deeplearning4j-modelimport/.../keras/preprocessors/ReshapePreprocessor.java``).
    ``targetShape`` is the Keras one: channels last, without the batch axis, at most one ``-1``.  The network
    keeps activations channels first, so the activation is put into the Keras order, reshaped, and put back."""
    JAVA = "ReshapePreprocessor"; FIELDS = ("targetShape",)
    def __init__(self, targetShape):
        self.targetShape = [int(v) for v in targetShape]
    def preProcess(self, x, minibatch=None, ctx=None):
        y = _to_channels_last(x).reshape([x.shape[0]] + self.targetShape)
        return _to_channels_first(y).contiguous()
    def output_type(self, it):
        src = _channels_last_shape(it)
        tgt = list(self.targetShape)
        if -1 in tgt:
            total, known = 1, 1
            for v in src:
                total *= v
            for v in tgt:
                known *= v if v != -1 else 1
            tgt[tgt.index(-1)] = total // known
        return _type_of_channels_last(tgt)
    def to_json(self):
        return {"@class": "org.deeplearning4j.nn.modelimport.keras.preprocessors." + self.JAVA, "targetShape": self.targetShape}


class PermutePreprocessor(InputPreProcessor):
    """Keras ``Permute`` (``.../keras/preprocessors/PermutePreprocessor.java``): ``dims`` are the 1-based Keras axes
    (channels last) in their new order."""
    JAVA = "PermutePreprocessor"; FIELDS = ("permutationIndices",)
    def __init__(self, permutationIndices):
        self.permutationIndices = [int(v) for v in permutationIndices]
    def preProcess(self, x, minibatch=None, ctx=None):
        y = _to_channels_last(x).permute(0, *self.permutationIndices)
        return _to_channels_first(y).contiguous()
    def output_type(self, it):
        src = _channels_last_shape(it)
        return _type_of_channels_last([src[i - 1] for i in self.permutationIndices])
    def to_json(self):
        return {"@class": "org.deeplearning4j.nn.modelimport.keras.preprocessors." + self.JAVA, "permutationIndices": self.permutationIndices}


PREPROCESSORS = {c.JAVA: c for c in (ReshapePreprocessor, PermutePreprocessor, CnnToFeedForwardPreProcessor, FeedForwardToCnnPreProcessor,
                                     Cnn3DToFeedForwardPreProcessor, FeedForwardToCnn3DPreProcessor,
                                     RnnToFeedForwardPreProcessor, FeedForwardToRnnPreProcessor,
                                     CnnToRnnPreProcessor, RnnToCnnPreProcessor, ComposableInputPreProcessor)}


def preprocessor_from_json(d):
    if d is None:
        return None
    cls = PREPROCESSORS[d["@class"].rsplit(".", 1)[-1]]
    if cls is ComposableInputPreProcessor:
        return cls([preprocessor_from_json(e) for e in d["inputPreProcessors"]])
    return cls(**{k: v for k, v in d.items() if k in cls.FIELDS})
