"""Model zoo (``deeplearning4j-zoo/src/main/java/org/deeplearning4j/zoo/model/*.java``).

Each ``ZooModel`` builds the same architecture as its reference class through the public
configuration API.  ``ResNet50`` reproduces the reference graph literally, including its quirks
(``ResNet50.java:178-241``: stride-2 conv block in stage 2, a 3x3 *max* pool named "avgpool",
l1 1e-7 / l2 5e-5).  Pre-trained weights are not downloadable here; ``initPretrained`` loads a
checkpoint from a local path instead.
"""
from __future__ import annotations

from ..nn.activations import Activation
from ..nn.conf.base import BackpropType, ConvolutionMode, InputType, PoolingType
from ..nn.conf.graphconf import ElementWiseVertex, MergeVertex
from ..nn.conf.neuralnet import NeuralNetConfiguration
from ..nn.layers.conv import (BatchNormalization, ConvolutionLayer, GlobalPoolingLayer, LocalResponseNormalization,
                              SeparableConvolution2D, SubsamplingLayer, Upsampling2D, ZeroPaddingLayer, Cropping2D,
                              SpaceToDepthLayer, DepthwiseConvolution2D)
from ..nn.layers.core import ActivationLayer, DenseLayer, DropoutLayer, OutputLayer, RnnOutputLayer, LossLayer
from ..nn.layers.recurrent import LSTM
from ..nn.updaters import Adam, AdaDelta, Nesterovs, RmsProp, Sgd
from ..nn.weights import NormalDistribution, WeightInit


class ZooModel:
    def __init__(self, numClasses=1000, seed=1234, inputShape=None, updater=None, weightInit=None, cacheMode="NONE",
                 workspaceMode="ENABLED", computeDataType=None, **kw):
        self.numClasses, self.seed = numClasses, seed
        self.inputShape = list(inputShape) if inputShape is not None else list(self.DEFAULT_INPUT)
        self.updater = updater or self.default_updater()
        self.weightInit = weightInit or self.DEFAULT_WEIGHT_INIT
        self.computeDataType = computeDataType
        self.__dict__.update(kw)

    DEFAULT_INPUT = (3, 224, 224)
    DEFAULT_WEIGHT_INIT = "XAVIER"

    def default_updater(self):
        return Nesterovs(0.1, 0.9)

    @classmethod
    def builder(cls):
        return _ZooBuilder(cls)

    def _base(self):
        b = NeuralNetConfiguration.Builder().seed(self.seed).updater(self.updater).weightInit(self.weightInit)
        if self.computeDataType is not None:
            b.computeDataType(self.computeDataType)
        return b

    def conf(self):
        raise NotImplementedError

    def init(self, device=None):
        from ..nn.conf.graphconf import ComputationGraphConfiguration
        from ..nn.graph import ComputationGraph
        from ..nn.multilayer import MultiLayerNetwork
        c = self.conf()
        net = ComputationGraph(c) if isinstance(c, ComputationGraphConfiguration) else MultiLayerNetwork(c)
        if device is not None:
            import torch
            net.device = torch.device(device)
        return net.init()

    def initPretrained(self, path=None, pretrainedType="IMAGENET"):
        if path is None:
            raise IOError("pretrained weights cannot be downloaded in this environment; pass a local checkpoint path")
        from ..nn.serializer import ModelGuesser
        return ModelGuesser.loadModelGuess(path)

    def metaData(self):
        return {"inputShape": [self.inputShape], "numOutputs": 1, "zooType": "CNN"}

    def modelType(self):
        return type(self).__name__


class _ZooBuilder:
    def __init__(self, cls):
        self._cls, self._kw = cls, {}

    def __getattr__(self, k):
        if k.startswith("_"):
            raise AttributeError(k)

        def s(*v):
            self._kw[k] = v[0] if len(v) == 1 else list(v)
            return self
        return s

    def build(self):
        return self._cls(**self._kw)


# ----------------------------------------------------------------------------- ResNet-50
class ResNet50(ZooModel):
    # the reference default is a truncated normal (0, 0.5) (ResNet50.java:55), which diverges without pretrained weights
    # at the first steps of a from-scratch run; He initialisation ("RELU") is this zoo's default, the reference's is
    # available through ``weightInit=WeightInitDistribution(TruncatedNormalDistribution(0.0, 0.5))``
    DEFAULT_WEIGHT_INIT = "RELU"

    def default_updater(self):
        return RmsProp(0.1, 0.96, 0.001)

    def _identity(self, g, k, f, stage, block, inp):
        cn, bn, an, sn = (f"{p}{stage}{block}_branch" for p in ("res", "bn", "act", "short"))
        g.addLayer(cn + "2a", ConvolutionLayer([1, 1], nOut=f[0]), inp)
        g.addLayer(bn + "2a", BatchNormalization(), cn + "2a")
        g.addLayer(an + "2a", ActivationLayer("RELU"), bn + "2a")
        g.addLayer(cn + "2b", ConvolutionLayer(k, nOut=f[1], convolutionMode=ConvolutionMode.Same), an + "2a")
        g.addLayer(bn + "2b", BatchNormalization(), cn + "2b")
        g.addLayer(an + "2b", ActivationLayer("RELU"), bn + "2b")
        g.addLayer(cn + "2c", ConvolutionLayer([1, 1], nOut=f[2]), an + "2b")
        g.addLayer(bn + "2c", BatchNormalization(), cn + "2c")
        g.addVertex(sn, ElementWiseVertex("Add"), bn + "2c", inp)
        g.addLayer(cn, ActivationLayer("RELU"), sn)

    def _conv(self, g, k, f, stage, block, inp, stride=(2, 2)):
        cn, bn, an, sn = (f"{p}{stage}{block}_branch" for p in ("res", "bn", "act", "short"))
        g.addLayer(cn + "2a", ConvolutionLayer([1, 1], list(stride), nOut=f[0]), inp)
        g.addLayer(bn + "2a", BatchNormalization(), cn + "2a")
        g.addLayer(an + "2a", ActivationLayer("RELU"), bn + "2a")
        g.addLayer(cn + "2b", ConvolutionLayer(k, nOut=f[1], convolutionMode=ConvolutionMode.Same), an + "2a")
        g.addLayer(bn + "2b", BatchNormalization(), cn + "2b")
        g.addLayer(an + "2b", ActivationLayer("RELU"), bn + "2b")
        g.addLayer(cn + "2c", ConvolutionLayer([1, 1], nOut=f[2]), an + "2b")
        g.addLayer(bn + "2c", BatchNormalization(), cn + "2c")
        g.addLayer(cn + "1", ConvolutionLayer([1, 1], list(stride), nOut=f[2]), inp)
        g.addLayer(bn + "1", BatchNormalization(), cn + "1")
        g.addVertex(sn, ElementWiseVertex("Add"), bn + "2c", bn + "1")
        g.addLayer(cn, ActivationLayer("RELU"), sn)

    def conf(self):
        c, h, w = self.inputShape
        g = (self._base().activation("IDENTITY").l1(1e-7).l2(5e-5).convolutionMode(ConvolutionMode.Truncate).graphBuilder())
        g.addInputs("input").setInputTypes(InputType.convolutional(h, w, c))
        g.addLayer("stem-zero", ZeroPaddingLayer(3, 3), "input")
        g.addLayer("stem-cnn1", ConvolutionLayer([7, 7], [2, 2], nOut=64), "stem-zero")
        g.addLayer("stem-batch1", BatchNormalization(), "stem-cnn1")
        g.addLayer("stem-act1", ActivationLayer("RELU"), "stem-batch1")
        g.addLayer("stem-maxpool1", SubsamplingLayer(PoolingType.MAX, [3, 3], [2, 2]), "stem-act1")
        k = [3, 3]
        self._conv(g, k, [64, 64, 256], "2", "a", "stem-maxpool1", (2, 2))
        self._identity(g, k, [64, 64, 256], "2", "b", "res2a_branch")
        self._identity(g, k, [64, 64, 256], "2", "c", "res2b_branch")
        self._conv(g, k, [128, 128, 512], "3", "a", "res2c_branch")
        for b, prev in zip("bcd", "abc"):
            self._identity(g, k, [128, 128, 512], "3", b, f"res3{prev}_branch")
        self._conv(g, k, [256, 256, 1024], "4", "a", "res3d_branch")
        for b, prev in zip("bcdef", "abcde"):
            self._identity(g, k, [256, 256, 1024], "4", b, f"res4{prev}_branch")
        self._conv(g, k, [512, 512, 2048], "5", "a", "res4f_branch")
        self._identity(g, k, [512, 512, 2048], "5", "b", "res5a_branch")
        self._identity(g, k, [512, 512, 2048], "5", "c", "res5b_branch")
        g.addLayer("avgpool", SubsamplingLayer(PoolingType.MAX, [3, 3]), "res5c_branch")
        g.addLayer("output", OutputLayer("NEGATIVELOGLIKELIHOOD", nOut=self.numClasses, activation="SOFTMAX"), "avgpool")
        g.setOutputs("output")
        return g.build()


# ----------------------------------------------------------------------------- text generation LSTM
class TextGenerationLSTM(ZooModel):
    """``TextGenerationLSTM.java:76-97``: 2 x LSTM(256, tanh) + RnnOutput(MCXENT, softmax), tBPTT 50."""
    DEFAULT_INPUT = (50, 77)          # [maxLength, totalUniqueCharacters]

    def __init__(self, totalUniqueCharacters=None, hidden=256, layers=2, tbptt=50, **kw):
        super().__init__(**kw)
        self.totalUniqueCharacters = totalUniqueCharacters or self.inputShape[1]
        self.hidden, self.layers, self.tbptt = hidden, layers, tbptt

    def default_updater(self):
        return RmsProp(0.01)

    def conf(self):
        lb = self._base().l2(0.001).list()
        n_in = self.totalUniqueCharacters
        for i in range(self.layers):
            lb.layer(LSTM(nIn=n_in, nOut=self.hidden, activation="TANH"))
            n_in = self.hidden
        lb.layer(RnnOutputLayer("MCXENT", nIn=n_in, nOut=self.totalUniqueCharacters, activation="SOFTMAX"))
        return lb.backpropType(BackpropType.TruncatedBPTT).tBPTTForwardLength(self.tbptt).tBPTTBackwardLength(self.tbptt).build()

    def metaData(self):
        return {"inputShape": [self.inputShape], "numOutputs": 1, "zooType": "RNN"}
