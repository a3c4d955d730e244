"""The rest of the model zoo (``deeplearning4j-zoo/.../zoo/model``): LeNet, SimpleCNN, AlexNet, VGG16, VGG19,
Darknet19, TinyYOLO, YOLO2, SqueezeNet, UNet, Xception, InceptionResNetV1, FaceNetNN4Small2 and NASNet,
each built through the public configuration API with the reference's layer names, so parameter keys of a
checkpoint line up with the reference's."""
from __future__ import annotations

import math

from ..nn.activations import Activation, ActivationLReLU
from ..nn.conf.base import ConvolutionMode, GradientNormalization, InputType, PoolingType
from ..nn.conf.graphconf import ElementWiseVertex, L2NormalizeVertex, MergeVertex, ScaleVertex
from ..nn.layers.conv import (BatchNormalization, ConvolutionLayer, Cropping2D, GlobalPoolingLayer, LocalResponseNormalization,
                              SeparableConvolution2D, SpaceToDepthLayer, SubsamplingLayer, Upsampling2D, ZeroPaddingLayer)
from ..nn.layers.core import ActivationLayer, CenterLossOutputLayer, CnnLossLayer, DenseLayer, DropoutLayer, LossLayer, OutputLayer
from ..nn.layers.special import Yolo2OutputLayer
from ..nn.updaters import AdaDelta, Adam, Nesterovs, RmsProp
from ..nn.weights import NormalDistribution
from .zoo import ZooModel

Same, Truncate = ConvolutionMode.Same, ConvolutionMode.Truncate


def _conv(k, s=(1, 1), p=(0, 0), **kw):
    return ConvolutionLayer(list(k), list(s), list(p), **kw)


def _pool(kind, k, s=None, p=(0, 0), **kw):
    return SubsamplingLayer(kind, list(k), list(s if s is not None else k), list(p), **kw)


# ----------------------------------------------------------------------------- LeNet / SimpleCNN / AlexNet
class LeNet(ZooModel):
    """``LeNet.java``: conv5x5(20) - max2 - conv5x5(50) - max2 - dense(500) - softmax, Same mode, flat MNIST-style input."""
    DEFAULT_INPUT = (1, 28, 28)

    def __init__(self, numClasses=10, **kw): super().__init__(numClasses=numClasses, **kw)
    def default_updater(self): return AdaDelta()

    def conf(self):
        c, h, w = self.inputShape
        return (self._base().activation("IDENTITY").convolutionMode(Same).list()
                .layer(_conv((5, 5), nIn=c, nOut=20, activation="RELU", layerName="cnn1"))
                .layer(_pool("MAX", (2, 2), (2, 2), layerName="maxpool1"))
                .layer(_conv((5, 5), nOut=50, activation="RELU", layerName="cnn2"))
                .layer(_pool("MAX", (2, 2), (2, 2), layerName="maxpool2"))
                .layer(DenseLayer(nOut=500, activation="RELU", layerName="ffn1"))
                .layer(OutputLayer("MCXENT", nOut=self.numClasses, activation="SOFTMAX", layerName="output"))
                .setInputType(InputType.convolutionalFlat(h, w, c)).build())


class SimpleCNN(ZooModel):
    DEFAULT_INPUT = (3, 48, 48)
    DEFAULT_WEIGHT_INIT = "RELU"
    def default_updater(self): return AdaDelta()

    def conf(self):
        c, h, w = self.inputShape
        lb = self._base().activation("IDENTITY").convolutionMode(Same).list()
        lb.layer(_conv((7, 7), nIn=c, nOut=16, layerName="image_array")).layer(BatchNormalization())
        lb.layer(_conv((7, 7), nIn=16, nOut=16)).layer(BatchNormalization()).layer(ActivationLayer("RELU"))
        lb.layer(_pool("AVG", (2, 2), (2, 2))).layer(DropoutLayer(0.5))
        for k, n in ((5, 32), (3, 64), (3, 128)):
            lb.layer(_conv((k, k), nOut=n)).layer(BatchNormalization()).layer(_conv((k, k), nOut=n)).layer(BatchNormalization())
            lb.layer(ActivationLayer("RELU")).layer(_pool("AVG", (2, 2), (2, 2))).layer(DropoutLayer(0.5))
        lb.layer(_conv((3, 3), nOut=256)).layer(BatchNormalization()).layer(_conv((3, 3), nOut=self.numClasses))
        lb.layer(GlobalPoolingLayer("AVG")).layer(ActivationLayer("SOFTMAX"))
        return lb.setInputType(InputType.convolutional(h, w, c)).validateOutputLayerConfig(False).build()


class AlexNet(ZooModel):
    DEFAULT_INPUT = (3, 224, 224)
    def default_updater(self): return Nesterovs(1e-2, 0.9)

    def conf(self):
        c, h, w = self.inputShape
        b = (self._base().weightInit(NormalDistribution(0.0, 0.01)).activation("RELU").biasUpdater(Nesterovs(2e-2, 0.9)).convolutionMode(Same)
             .gradientNormalization(GradientNormalization.RenormalizeL2PerLayer).l2(5e-4).miniBatch(False))
        d005 = NormalDistribution(0, 0.005)
        return (b.list()
                .layer(_conv((11, 11), (4, 4), nIn=c, nOut=96, convolutionMode=Truncate, layerName="cnn1"))
                .layer(LocalResponseNormalization())
                .layer(_pool("MAX", (3, 3), (2, 2), (1, 1), layerName="maxpool1"))
                .layer(_conv((5, 5), (1, 1), (2, 2), nOut=256, convolutionMode=Truncate, biasInit=1.0, layerName="cnn2"))
                .layer(_pool("MAX", (3, 3), (2, 2), convolutionMode=Truncate, layerName="maxpool2"))
                .layer(LocalResponseNormalization())
                .layer(_conv((3, 3), nOut=384, convolutionMode=Same, layerName="cnn3"))
                .layer(_conv((3, 3), nOut=384, biasInit=1.0, layerName="cnn4"))
                .layer(_conv((3, 3), nOut=256, biasInit=1.0, layerName="cnn5"))
                .layer(_pool("MAX", (3, 3), (2, 2), convolutionMode=Truncate, layerName="maxpool3"))
                .layer(DenseLayer(nOut=4096, weightInit=d005, biasInit=1.0, layerName="ffn1"))
                .layer(DenseLayer(nOut=4096, weightInit=d005, biasInit=1.0, dropOut=0.5, layerName="ffn2"))
                .layer(OutputLayer("NEGATIVELOGLIKELIHOOD", nOut=self.numClasses, activation="SOFTMAX", weightInit=d005, biasInit=0.1, layerName="output"))
                .setInputType(InputType.convolutional(h, w, c)).build())


# ----------------------------------------------------------------------------- VGG
class VGG16(ZooModel):
    BLOCKS = ((64, 2), (128, 2), (256, 3), (512, 3), (512, 3))
    def default_updater(self): return Nesterovs(1e-2, 0.9)

    def conf(self):
        c, h, w = self.inputShape
        g = self._base().activation("RELU").graphBuilder().addInputs("in")
        prev, i = "in", 0
        for n, reps in self.BLOCKS:
            for _ in range(reps):
                g.addLayer(str(i), _conv((3, 3), (1, 1), (1, 1), nOut=n, **({"nIn": c} if i == 0 else {})), prev)
                prev, i = str(i), i + 1
            g.addLayer(str(i), _pool("MAX", (2, 2), (2, 2)), prev)
            prev, i = str(i), i + 1
        for _ in range(2):
            g.addLayer(str(i), DenseLayer(nOut=4096, dropOut=0.5), prev)
            prev, i = str(i), i + 1
        g.addLayer(str(i), OutputLayer("NEGATIVELOGLIKELIHOOD", nOut=self.numClasses, activation="SOFTMAX", layerName="output"), prev)
        return g.setOutputs(str(i)).setInputTypes(InputType.convolutionalFlat(h, w, c)).build()


class VGG19(VGG16):
    BLOCKS = ((64, 2), (128, 2), (256, 4), (512, 4), (512, 4))


# ----------------------------------------------------------------------------- Darknet family
def _dark(g, n, k, n_in, n_out, pool, pool_stride=None, inp=None):
    """``DarknetHelper.addLayers``: conv (no bias, Same) - BN - LeakyReLU(0.1) [- max pool]."""
    if inp is None:
        for cand in (f"maxpooling2d_{n - 1}", f"activation_{n - 1}", f"concatenate_{n - 1}", "input"):
            if cand in g.getVertices() or cand == "input":
                inp = cand
                break
    g.addLayer(f"convolution2d_{n}", _conv((k, k), nIn=n_in, nOut=n_out, weightInit="XAVIER", convolutionMode=Same, hasBias=False, activation="IDENTITY"), inp)
    g.addLayer(f"batchnormalization_{n}", BatchNormalization(nIn=n_out, nOut=n_out, weightInit="XAVIER", activation="IDENTITY"), f"convolution2d_{n}")
    g.addLayer(f"activation_{n}", ActivationLayer(ActivationLReLU(alpha=0.1)), f"batchnormalization_{n}")
    if pool > 0:
        ps = pool if pool_stride is None else pool_stride
        g.addLayer(f"maxpooling2d_{n}", SubsamplingLayer("MAX", [pool, pool], [ps, ps], convolutionMode=Same), f"activation_{n}")
    return g


_DARK19 = [(3, 32, 2), (3, 64, 2), (3, 128, 0), (1, 64, 0), (3, 128, 2), (3, 256, 0), (1, 128, 0), (3, 256, 2), (3, 512, 0), (1, 256, 0),
           (3, 512, 0), (1, 256, 0), (3, 512, 2), (3, 1024, 0), (1, 512, 0), (3, 1024, 0), (1, 512, 0), (3, 1024, 0)]


class Darknet19(ZooModel):
    DEFAULT_INPUT = (3, 224, 224)
    def default_updater(self): return Nesterovs(1e-3, 0.9)

    def _trunk(self, g, c):
        n_in = c
        for i, (k, n_out, pool) in enumerate(_DARK19, start=1):
            _dark(g, i, k, n_in, n_out, pool)
            n_in = n_out

    def conf(self):
        c, h, w = self.inputShape
        g = self._base().l2(1e-5).activation("IDENTITY").graphBuilder().addInputs("input").setInputTypes(InputType.convolutional(h, w, c))
        self._trunk(g, c)
        g.addLayer("convolution2d_19", _conv((1, 1), nIn=1024, nOut=self.numClasses, convolutionMode=Same, weightInit="RELU", activation="IDENTITY"), "activation_18")
        g.addLayer("globalpooling", GlobalPoolingLayer("AVG"), "convolution2d_19")
        g.addLayer("softmax", ActivationLayer("SOFTMAX"), "globalpooling")
        g.addLayer("loss", LossLayer("NEGATIVELOGLIKELIHOOD", activation="IDENTITY"), "softmax")
        return g.setOutputs("loss").validateOutputLayerConfig(False).build()


class TinyYOLO(ZooModel):
    DEFAULT_INPUT = (3, 416, 416)
    PRIORS = [[1.08, 1.19], [3.42, 4.41], [6.63, 11.38], [9.42, 5.11], [16.62, 10.52]]

    def __init__(self, numClasses=20, priorBoxes=None, **kw):
        super().__init__(numClasses=numClasses, **kw)
        self.priorBoxes = priorBoxes or self.PRIORS
        self.nBoxes = len(self.priorBoxes)

    def default_updater(self): return Adam(1e-3)

    def _builder(self):
        c, h, w = self.inputShape
        return (self._base().gradientNormalization(GradientNormalization.RenormalizeL2PerLayer).gradientNormalizationThreshold(1.0).l2(1e-5)
                .activation("IDENTITY").graphBuilder().addInputs("input").setInputTypes(InputType.convolutional(h, w, c)))

    def conf(self):
        g = self._builder()
        n_in = self.inputShape[0]
        for i, (n_out, pool, ps) in enumerate([(16, 2, 2), (32, 2, 2), (64, 2, 2), (128, 2, 2), (256, 2, 2), (512, 2, 1), (1024, 0, 0), (1024, 0, 0)], start=1):
            _dark(g, i, 3, n_in, n_out, pool, ps)
            n_in = n_out
        g.addLayer("convolution2d_9", _conv((1, 1), nIn=1024, nOut=self.nBoxes * (5 + self.numClasses), convolutionMode=Same, weightInit="RELU", activation="IDENTITY"), "activation_8")
        g.addLayer("outputs", Yolo2OutputLayer(boundingBoxes=self.priorBoxes), "convolution2d_9")
        return g.setOutputs("outputs").build()

    @staticmethod
    def getGridWidth(inputShape): return inputShape[1] // 32
    @staticmethod
    def getGridHeight(inputShape): return inputShape[2] // 32


class YOLO2(TinyYOLO):
    DEFAULT_INPUT = (3, 608, 608)
    PRIORS = [[0.57273, 0.677385], [1.87446, 2.06253], [3.33843, 5.47434], [7.88282, 3.52778], [9.77052, 9.16828]]

    def __init__(self, numClasses=80, **kw): super().__init__(numClasses=numClasses, **kw)

    def conf(self):
        g = self._builder()
        n_in = self.inputShape[0]
        for i, (k, n_out, pool) in enumerate(_DARK19, start=1):
            _dark(g, i, k, n_in, n_out, pool)
            n_in = n_out
        _dark(g, 19, 3, 1024, 1024, 0)
        _dark(g, 20, 3, 1024, 1024, 0)
        _dark(g, 21, 1, 512, 64, 0, 0, inp="activation_13")
        g.addLayer("rearrange_21", SpaceToDepthLayer(2), "activation_21")
        g.addVertex("concatenate_21", MergeVertex(), "rearrange_21", "activation_20")
        _dark(g, 22, 3, 1024 + 256, 1024, 0, 0, inp="concatenate_21")
        g.addLayer("convolution2d_23", _conv((1, 1), nIn=1024, nOut=self.nBoxes * (5 + self.numClasses), convolutionMode=Same, weightInit="RELU", activation="IDENTITY"), "activation_22")
        g.addLayer("outputs", Yolo2OutputLayer(boundingBoxes=self.priorBoxes), "convolution2d_23")
        return g.setOutputs("outputs").build()


# ----------------------------------------------------------------------------- SqueezeNet / UNet / Xception
class SqueezeNet(ZooModel):
    DEFAULT_INPUT = (3, 227, 227)
    DEFAULT_WEIGHT_INIT = "RELU"
    def default_updater(self): return Adam(1e-3)

    @staticmethod
    def _fire(g, i, sq, ex, inp):
        p = f"fire{i}"
        g.addLayer(p + "_sq1x1", _conv((1, 1), nOut=sq), inp).addLayer(p + "_relu_sq1x1", ActivationLayer("RELU"), p + "_sq1x1")
        g.addLayer(p + "_exp1x1", _conv((1, 1), nOut=ex), p + "_relu_sq1x1").addLayer(p + "_relu_exp1x1", ActivationLayer("RELU"), p + "_exp1x1")
        g.addLayer(p + "_exp3x3", _conv((3, 3), nOut=ex, convolutionMode=Same), p + "_relu_sq1x1").addLayer(p + "_relu_exp3x3", ActivationLayer("RELU"), p + "_exp3x3")
        g.addVertex(p, MergeVertex(), p + "_relu_exp1x1", p + "_relu_exp3x3")
        return p

    def conf(self):
        c, h, w = self.inputShape
        g = self._base().l2(5e-5).convolutionMode(Truncate).graphBuilder().addInputs("input").setInputTypes(InputType.convolutional(h, w, c))
        g.addLayer("conv1", _conv((3, 3), (2, 2), nOut=64), "input").addLayer("conv1_act", ActivationLayer("RELU"), "conv1")
        g.addLayer("pool1", _pool("MAX", (3, 3), (2, 2)), "conv1_act")
        self._fire(g, 2, 16, 64, "pool1"); self._fire(g, 3, 16, 64, "fire2")
        g.addLayer("pool3", _pool("MAX", (3, 3), (2, 2)), "fire3")
        self._fire(g, 4, 32, 128, "pool3"); self._fire(g, 5, 32, 128, "fire4")
        g.addLayer("pool5", _pool("MAX", (3, 3), (2, 2)), "fire5")
        self._fire(g, 6, 48, 192, "pool5"); self._fire(g, 7, 48, 192, "fire6"); self._fire(g, 8, 64, 256, "fire7"); self._fire(g, 9, 64, 256, "fire8")
        g.addLayer("drop9", DropoutLayer(0.5), "fire9").addLayer("conv10", _conv((1, 1), nOut=self.numClasses), "drop9")
        g.addLayer("conv10_act", ActivationLayer("RELU"), "conv10").addLayer("avg_pool", GlobalPoolingLayer("AVG"), "conv10_act")
        g.addLayer("softmax", ActivationLayer("SOFTMAX"), "avg_pool").addLayer("loss", LossLayer("MCXENT", activation="IDENTITY"), "softmax")
        return g.setOutputs("loss").validateOutputLayerConfig(False).build()


class UNet(ZooModel):
    DEFAULT_INPUT = (3, 512, 512)
    DEFAULT_WEIGHT_INIT = "RELU"

    def __init__(self, numClasses=1, **kw): super().__init__(numClasses=numClasses, **kw)
    def default_updater(self): return AdaDelta()

    def conf(self):
        c, h, w = self.inputShape
        g = self._base().l2(5e-5).graphBuilder().addInputs("input").setInputTypes(InputType.convolutional(h, w, c))
        cv = lambda n, k=3, act="RELU": _conv((k, k), nOut=n, convolutionMode=Same, activation=act)
        prev = "input"
        for i, n in enumerate((64, 128, 256, 512), start=1):
            g.addLayer(f"conv{i}-1", cv(n), prev).addLayer(f"conv{i}-2", cv(n), f"conv{i}-1")
            last = f"conv{i}-2"
            if i == 4:
                g.addLayer("drop4", DropoutLayer(0.5), last)
                last = "drop4"
            g.addLayer(f"pool{i}", _pool("MAX", (2, 2)), last)
            prev = f"pool{i}"
        g.addLayer("conv5-1", cv(1024), "pool4").addLayer("conv5-2", cv(1024), "conv5-1").addLayer("drop5", DropoutLayer(0.5), "conv5-2")
        prev = "drop5"
        for i, (n, skip) in enumerate(((512, "drop4"), (256, "conv3-2"), (128, "conv2-2"), (64, "conv1-2")), start=6):
            g.addLayer(f"up{i}-1", Upsampling2D(2), prev).addLayer(f"up{i}-2", cv(n, 2), f"up{i}-1")
            g.addVertex(f"merge{i}", MergeVertex(), skip, f"up{i}-2")
            g.addLayer(f"conv{i}-1", cv(n), f"merge{i}").addLayer(f"conv{i}-2", cv(n), f"conv{i}-1")
            prev = f"conv{i}-2"
        g.addLayer("conv9-3", cv(2), "conv9-2").addLayer("conv10", _conv((1, 1), nOut=1, convolutionMode=Same, activation="IDENTITY"), "conv9-3")
        g.addLayer("output", CnnLossLayer("XENT", activation="SIGMOID"), "conv10")
        return g.setOutputs("output").build()


class Xception(ZooModel):
    DEFAULT_INPUT = (3, 299, 299)
    DEFAULT_WEIGHT_INIT = "RELU"
    def default_updater(self): return AdaDelta()

    def conf(self):
        c, h, w = self.inputShape
        g = self._base().l2(4e-5).convolutionMode(Truncate).graphBuilder().addInputs("input").setInputTypes(InputType.convolutional(h, w, c))
        sep = lambda n: SeparableConvolution2D([3, 3], nOut=n, hasBias=False, convolutionMode=Same)
        relu = lambda: ActivationLayer("RELU")
        g.addLayer("block1_conv1", _conv((3, 3), (2, 2), nOut=32, hasBias=False), "input").addLayer("block1_conv1_bn", BatchNormalization(), "block1_conv1")
        g.addLayer("block1_conv1_act", relu(), "block1_conv1_bn")
        g.addLayer("block1_conv2", _conv((3, 3), nOut=64, hasBias=False), "block1_conv1_act").addLayer("block1_conv2_bn", BatchNormalization(), "block1_conv2")
        g.addLayer("block1_conv2_act", relu(), "block1_conv2_bn")
        g.addLayer("residual1_conv", _conv((1, 1), (2, 2), nOut=128, hasBias=False, convolutionMode=Same), "block1_conv2_act").addLayer("residual1", BatchNormalization(), "residual1_conv")
        g.addLayer("block2_sepconv1", sep(128), "block1_conv2_act").addLayer("block2_sepconv1_bn", BatchNormalization(), "block2_sepconv1")
        g.addLayer("block2_sepconv1_act", relu(), "block2_sepconv1_bn")
        g.addLayer("block2_sepconv2", sep(128), "block2_sepconv1_act").addLayer("block2_sepconv2_bn", BatchNormalization(), "block2_sepconv2")
        g.addLayer("block2_pool", _pool("MAX", (3, 3), (2, 2), convolutionMode=Same), "block2_sepconv2_bn")
        g.addVertex("add1", ElementWiseVertex("Add"), "block2_pool", "residual1")
        for blk, n, add in ((3, 256, 1), (4, 728, 2)):
            g.addLayer(f"residual{add + 1}_conv", _conv((1, 1), (2, 2), nOut=n, hasBias=False, convolutionMode=Same), f"add{add}")
            g.addLayer(f"residual{add + 1}", BatchNormalization(), f"residual{add + 1}_conv")
            g.addLayer(f"block{blk}_sepconv1_act", relu(), f"add{add}").addLayer(f"block{blk}_sepconv1", sep(n), f"block{blk}_sepconv1_act")
            g.addLayer(f"block{blk}_sepconv1_bn", BatchNormalization(), f"block{blk}_sepconv1")
            g.addLayer(f"block{blk}_sepconv2_act", relu(), f"block{blk}_sepconv1_bn").addLayer(f"block{blk}_sepconv2", sep(n), f"block{blk}_sepconv2_act")
            g.addLayer(f"block{blk}_sepconv2_bn", BatchNormalization(), f"block{blk}_sepconv2")
            g.addLayer(f"block{blk}_pool", _pool("MAX", (3, 3), (2, 2), convolutionMode=Same), f"block{blk}_sepconv2_bn")
            g.addVertex(f"add{add + 1}", ElementWiseVertex("Add"), f"block{blk}_pool", f"residual{add + 1}")
        residual = 3
        for blk in range(5, 13):
            prev, b = f"add{residual}", f"block{blk}"
            last = prev
            for j in (1, 2, 3):
                g.addLayer(f"{b}_sepconv{j}_act", relu(), last).addLayer(f"{b}_sepconv{j}", sep(728), f"{b}_sepconv{j}_act")
                g.addLayer(f"{b}_sepconv{j}_bn", BatchNormalization(), f"{b}_sepconv{j}")
                last = f"{b}_sepconv{j}_bn"
            g.addVertex(f"add{residual + 1}", ElementWiseVertex("Add"), last, prev)
            residual += 1
        g.addLayer("residual12_conv", _conv((1, 1), (2, 2), nOut=1024, hasBias=False, convolutionMode=Same), f"add{residual}")
        g.addLayer("residual12", BatchNormalization(), "residual12_conv")
        g.addLayer("block13_sepconv1_act", relu(), "add11").addLayer("block13_sepconv1", sep(728), "block13_sepconv1_act")
        g.addLayer("block13_sepconv1_bn", BatchNormalization(), "block13_sepconv1")
        g.addLayer("block13_sepconv2_act", relu(), "block13_sepconv1_bn").addLayer("block13_sepconv2", sep(1024), "block13_sepconv2_act")
        g.addLayer("block13_sepconv2_bn", BatchNormalization(), "block13_sepconv2")
        g.addLayer("block13_pool", _pool("MAX", (3, 3), (2, 2), convolutionMode=Same), "block13_sepconv2_bn")
        g.addVertex("add12", ElementWiseVertex("Add"), "block13_pool", "residual12")
        g.addLayer("block14_sepconv1", sep(1536), "add12").addLayer("block14_sepconv1_bn", BatchNormalization(), "block14_sepconv1")
        g.addLayer("block14_sepconv1_act", relu(), "block14_sepconv1_bn")
        g.addLayer("block14_sepconv2", sep(2048), "block14_sepconv1_act").addLayer("block14_sepconv2_bn", BatchNormalization(), "block14_sepconv2")
        g.addLayer("block14_sepconv2_act", relu(), "block14_sepconv2_bn").addLayer("avg_pool", GlobalPoolingLayer("AVG"), "block14_sepconv2_act")
        g.addLayer("predictions", OutputLayer("MCXENT", nOut=self.numClasses, activation="SOFTMAX"), "avg_pool")
        return g.setOutputs("predictions").build()


# ----------------------------------------------------------------------------- Inception-ResNet v1 / FaceNet
def _bn(n=None, **kw):
    return BatchNormalization(decay=0.995, eps=0.001, **({"nIn": n, "nOut": n} if n else {}), **kw)


class InceptionResNetV1(ZooModel):
    DEFAULT_INPUT = (3, 160, 160)
    DEFAULT_WEIGHT_INIT = "RELU"
    def default_updater(self): return RmsProp(0.1, 0.96, 0.001)

    @staticmethod
    def _res(g, block, scale, act_scale, inp, n_in, branches, merge_n, pre_activation=False):
        """``InceptionResNetHelper.inceptionV1Res{A,B,C}``: ``branches`` is a list of conv chains [(kernel, nOut), ...]."""
        nm = lambda l, i: f"{block}-{l}-{i}"
        prev = inp
        if pre_activation:
            g.addLayer(nm("activation1", 0), ActivationLayer("TANH"), inp)
            prev = nm("activation1", 0)
        for i in range(1, scale + 1):
            k, ends = 1, []
            for chain in branches:
                last, last_n = prev, n_in
                for kernel, n_out in chain:
                    g.addLayer(nm(f"cnn{k}", i), _conv(kernel, nIn=last_n, nOut=n_out, convolutionMode=Same), last)
                    g.addLayer(nm(f"batch{k}", i), _bn(n_out), nm(f"cnn{k}", i))
                    last, last_n, k = nm(f"batch{k}", i), n_out, k + 1
                ends.append(last)
            g.addVertex(nm("merge1", i), MergeVertex(), *ends)
            g.addLayer(nm(f"cnn{k}", i), _conv(merge_n[0], nIn=merge_n[1], nOut=n_in, convolutionMode=Same), nm("merge1", i))
            g.addLayer(nm(f"batch{k}", i), _bn(n_in), nm(f"cnn{k}", i))
            g.addVertex(nm("scaling", i), ScaleVertex(act_scale), nm(f"batch{k}", i))
            g.addLayer(nm("shortcut-identity", i), ActivationLayer("IDENTITY"), prev)
            g.addVertex(nm("shortcut", i), ElementWiseVertex("Add"), nm("scaling", i), nm("shortcut-identity", i))
            name = block if i == scale else nm("activation", i)
            g.addLayer(name, ActivationLayer("TANH"), nm("shortcut", i))
            prev = name
        return g

    def graphBuilder(self, inp="input1"):
        c, h, w = self.inputShape
        g = self._base().activation("RELU").l2(5e-5).convolutionMode(Truncate).graphBuilder()
        g.addInputs(inp).setInputTypes(InputType.convolutional(h, w, c))
        stem = [("1", (3, 3), (2, 2), 32, Truncate), ("2", (3, 3), (1, 1), 32, Truncate), ("3", (3, 3), (1, 1), 64, Same)]
        prev, n_in = inp, c
        for s, k, st, n, mode in stem:
            g.addLayer(f"stem-cnn{s}", _conv(k, st, nIn=n_in, nOut=n, convolutionMode=mode), prev).addLayer(f"stem-batch{s}", _bn(n), f"stem-cnn{s}")
            prev, n_in = f"stem-batch{s}", n
        g.addLayer("stem-pool4", _pool("MAX", (3, 3), (2, 2)), prev)
        prev = "stem-pool4"
        for s, k, st, n in (("5", (1, 1), (1, 1), 80), ("6", (3, 3), (1, 1), 128), ("7", (3, 3), (2, 2), 192)):
            g.addLayer(f"stem-cnn{s}", _conv(k, st, nIn=n_in, nOut=n), prev).addLayer(f"stem-batch{s}", _bn(n), f"stem-cnn{s}")
            prev, n_in = f"stem-batch{s}", n
        self._res(g, "resnetA", 5, 0.17, prev, 192, [[((1, 1), 32)], [((1, 1), 32), ((3, 3), 32)], [((1, 1), 32), ((3, 3), 32), ((3, 3), 32)]], ((3, 3), 96))
        g.addLayer("reduceA-cnn1", _conv((3, 3), (2, 2), nIn=192, nOut=192), "resnetA").addLayer("reduceA-batch1", _bn(192), "reduceA-cnn1")
        g.addLayer("reduceA-cnn2", _conv((1, 1), nIn=192, nOut=128, convolutionMode=Same), "resnetA").addLayer("reduceA-batch2", _bn(128), "reduceA-cnn2")
        g.addLayer("reduceA-cnn3", _conv((3, 3), nIn=128, nOut=128, convolutionMode=Same), "reduceA-batch2").addLayer("reduceA-batch3", _bn(128), "reduceA-cnn3")
        g.addLayer("reduceA-cnn4", _conv((3, 3), (2, 2), nIn=128, nOut=192), "reduceA-batch3").addLayer("reduceA-batch4", _bn(192), "reduceA-cnn4")
        g.addLayer("reduceA-pool5", _pool("MAX", (3, 3), (2, 2)), "resnetA")
        g.addVertex("reduceA", MergeVertex(), "reduceA-batch1", "reduceA-batch4", "reduceA-pool5")
        self._res(g, "resnetB", 10, 0.10, "reduceA", 576, [[((1, 1), 128)], [((1, 1), 128), ((1, 3), 128), ((3, 1), 128)]], ((1, 1), 256), pre_activation=True)
        g.addLayer("reduceB-pool1", _pool("MAX", (3, 3), (2, 2)), "resnetB")
        k = 2
        outs = ["reduceB-pool1"]
        bi = 1
        for chain in ([((1, 1), (1, 1), Same), ((3, 3), (2, 2), Truncate)], [((1, 1), (1, 1), Same), ((3, 3), (2, 2), Truncate)],
                      [((1, 1), (1, 1), Same), ((3, 3), (1, 1), Same), ((3, 3), (2, 2), Truncate)]):
            last, n_in = "resnetB", 576
            for kernel, st, mode in chain:
                g.addLayer(f"reduceB-cnn{k}", _conv(kernel, st, nIn=n_in, nOut=256, convolutionMode=mode), last).addLayer(f"reduceB-batch{bi}", _bn(256), f"reduceB-cnn{k}")
                last, n_in, k, bi = f"reduceB-batch{bi}", 256, k + 1, bi + 1
            outs.append(last)
        g.addVertex("reduceB", MergeVertex(), *outs)
        self._res(g, "resnetC", 5, 0.20, "reduceB", 1344, [[((1, 1), 192)], [((1, 1), 192), ((1, 3), 192), ((3, 1), 192)]], ((1, 1), 384))
        g.addLayer("avgpool", _pool("AVG", (1, 1), (1, 1)), "resnetC")
        return g

    def conf(self):
        g = self.graphBuilder("input1")
        g.addLayer("bottleneck", DenseLayer(nOut=128), "avgpool")
        g.addVertex("embeddings", L2NormalizeVertex([1], 1e-10), "bottleneck")
        g.addLayer("outputLayer", CenterLossOutputLayer("NEGATIVELOGLIKELIHOOD", activation="SOFTMAX", alpha=0.9, lambda_=1e-4, nIn=128, nOut=self.numClasses), "embeddings")
        return g.setOutputs("outputLayer").build()


class FaceNetNN4Small2(ZooModel):
    DEFAULT_INPUT = (3, 96, 96)
    DEFAULT_WEIGHT_INIT = "RELU"

    def __init__(self, embeddingSize=128, transferFunction="RELU", **kw):
        super().__init__(**kw)
        self.embeddingSize, self.transferFunction = embeddingSize, transferFunction

    def default_updater(self): return Adam(0.1, 0.9, 0.999, 0.01)

    def _inception(self, g, name, n_in, kernels, strides, out_sizes, reduce_sizes, pool_type, inp, pnorm=0):
        """``FaceNetHelper.appendGraph``."""
        m, tf = f"inception-{name}", self.transferFunction
        ends = []
        for i, (k, s) in enumerate(zip(kernels, strides)):
            g.addLayer(f"{m}-cnn1-{i}", _conv((1, 1), nIn=n_in, nOut=reduce_sizes[i], biasInit=0.2), inp)
            g.addLayer(f"{m}-batch1-{i}", BatchNormalization(nIn=reduce_sizes[i], nOut=reduce_sizes[i]), f"{m}-cnn1-{i}")
            g.addLayer(f"{m}-transfer1-{i}", ActivationLayer(tf), f"{m}-batch1-{i}")
            pad = (s // 2) * 2
            g.addLayer(f"{m}-reduce1-{i}", _conv((k, k), (s, s), (pad, pad), nIn=reduce_sizes[i], nOut=out_sizes[i], biasInit=0.2), f"{m}-transfer1-{i}")
            g.addLayer(f"{m}-batch2-{i}", BatchNormalization(nIn=out_sizes[i], nOut=out_sizes[i]), f"{m}-reduce1-{i}")
            g.addLayer(f"{m}-transfer2-{i}", ActivationLayer(tf), f"{m}-batch2-{i}")
            ends.append(f"{m}-transfer2-{i}")
        i = len(kernels)
        if i < len(reduce_sizes):
            g.addLayer(f"{m}-pool1", SubsamplingLayer(pool_type, [3, 3], [1, 1], [1, 1], **({"pnorm": pnorm} if pool_type == "PNORM" else {})), inp)
            g.addLayer(f"{m}-cnn2", _conv((1, 1), nIn=n_in, nOut=reduce_sizes[i], biasInit=0.2), f"{m}-pool1")
            g.addLayer(f"{m}-batch3", BatchNormalization(nIn=reduce_sizes[i], nOut=reduce_sizes[i]), f"{m}-cnn2")
            g.addLayer(f"{m}-transfer3", ActivationLayer(tf), f"{m}-batch3")
            ends.append(f"{m}-transfer3")
        i += 1
        if i < len(reduce_sizes):
            g.addLayer(f"{m}-reduce2", _conv((1, 1), nIn=n_in, nOut=reduce_sizes[i], biasInit=0.2), inp)
            g.addLayer(f"{m}-batch4", BatchNormalization(nIn=reduce_sizes[i], nOut=reduce_sizes[i]), f"{m}-reduce2")
            g.addLayer(f"{m}-transfer4", ActivationLayer(tf), f"{m}-batch4")
            ends.append(f"{m}-transfer4")
        g.addVertex(m, MergeVertex(), *ends)

    def _reduction(self, g, name, n_in, a, b, inp):
        tf = self.transferFunction
        for prefix, (r, o), names in ((name, a, ("1x1", "transfer1", "3x3", "transfer2")), (f"{name}-2", b, ("1x1", "transfer3", "5x5", "transfer4"))):
            g.addLayer(f"{prefix}-{names[0]}", _conv((1, 1), nIn=n_in, nOut=r), inp).addLayer(f"{prefix}-{names[0]}-norm", BatchNormalization(nIn=r, nOut=r), f"{prefix}-{names[0]}")
            g.addLayer(f"{prefix}-{names[1]}", ActivationLayer(tf), f"{prefix}-{names[0]}-norm")
            g.addLayer(f"{prefix}-{names[2]}", _conv((3, 3), (2, 2), nIn=r, nOut=o), f"{prefix}-{names[1]}")
            g.addLayer(f"{prefix}-{names[2]}-norm", BatchNormalization(nIn=o, nOut=o), f"{prefix}-{names[2]}")
            g.addLayer(f"{prefix}-{names[3]}", ActivationLayer(tf), f"{prefix}-{names[2]}-norm")
        g.addLayer(f"{name}-pool", _pool("MAX", (3, 3), (2, 2), (1, 1)), inp)
        g.addVertex(f"inception-{name}", MergeVertex(), f"{name}-transfer2", f"{name}-2-transfer4", f"{name}-pool")

    def conf(self):
        c, h, w = self.inputShape
        tf = self.transferFunction
        g = (self._base().activation("IDENTITY").l2(5e-5).convolutionMode(Same).graphBuilder().addInputs("input1")
             .setInputTypes(InputType.convolutional(h, w, c)))
        g.addLayer("stem-cnn1", _conv((7, 7), (2, 2), (3, 3), nIn=c, nOut=64, convolutionMode=Truncate), "input1").addLayer("stem-batch1", BatchNormalization(nIn=64, nOut=64), "stem-cnn1")
        g.addLayer("stem-activation1", ActivationLayer("RELU"), "stem-batch1")
        g.addLayer("stem-pool1", _pool("MAX", (3, 3), (2, 2), (1, 1), convolutionMode=Truncate), "stem-activation1")
        g.addLayer("stem-lrn1", LocalResponseNormalization(k=1, n=5, alpha=1e-4, beta=0.75), "stem-pool1")
        g.addLayer("inception-2-cnn1", _conv((1, 1), nIn=64, nOut=64), "stem-lrn1").addLayer("inception-2-batch1", BatchNormalization(nIn=64, nOut=64), "inception-2-cnn1")
        g.addLayer("inception-2-activation1", ActivationLayer("RELU"), "inception-2-batch1")
        g.addLayer("inception-2-cnn2", _conv((3, 3), (1, 1), (1, 1), nIn=64, nOut=192, convolutionMode=Truncate), "inception-2-activation1")
        g.addLayer("inception-2-batch2", BatchNormalization(nIn=192, nOut=192), "inception-2-cnn2").addLayer("inception-2-activation2", ActivationLayer("RELU"), "inception-2-batch2")
        g.addLayer("inception-2-lrn1", LocalResponseNormalization(k=1, n=5, alpha=1e-4, beta=0.75), "inception-2-activation2")
        g.addLayer("inception-2-pool1", _pool("MAX", (3, 3), (2, 2), (1, 1), convolutionMode=Truncate), "inception-2-lrn1")
        T = Truncate
        sub = self._base().convolutionMode(T)
        del sub
        self._inception(g, "3a", 192, (3, 5), (1, 1), (128, 32), (96, 16, 32, 64), "MAX", "inception-2-pool1")
        self._inception(g, "3b", 256, (3, 5), (1, 1), (128, 64), (96, 32, 64, 64), "PNORM", "inception-3a", 2)
        self._reduction(g, "3c", 320, (128, 256), (32, 64), "inception-3b")
        self._inception(g, "4a", 640, (3, 5), (1, 1), (192, 64), (96, 32, 128, 256), "PNORM", "inception-3c", 2)
        self._reduction(g, "4e", 640, (160, 256), (64, 128), "inception-4a")
        for blk, n_in, pool in (("5a", 1024, "PNORM"), ("5b", 736, "MAX")):
            g.addLayer(f"{blk}-1x1", _conv((1, 1), nIn=n_in, nOut=256), f"inception-{'4e' if blk == '5a' else '5a'}")
            src = f"inception-{'4e' if blk == '5a' else '5a'}"
            g.addLayer(f"{blk}-1x1-norm", BatchNormalization(nIn=256, nOut=256), f"{blk}-1x1").addLayer(f"{blk}-transfer1", ActivationLayer(tf), f"{blk}-1x1-norm")
            g.addLayer(f"{blk}-2-1x1", _conv((1, 1), nIn=n_in, nOut=96), src).addLayer(f"{blk}-2-1x1-norm", BatchNormalization(nIn=96, nOut=96), f"{blk}-2-1x1")
            g.addLayer(f"{blk}-2-transfer2", ActivationLayer(tf), f"{blk}-2-1x1-norm")
            g.addLayer(f"{blk}-2-3x3", _conv((3, 3), nIn=96, nOut=384), f"{blk}-2-transfer2").addLayer(f"{blk}-2-3x3-norm", BatchNormalization(nIn=384, nOut=384), f"{blk}-2-3x3")
            g.addLayer(f"{blk}-2-transfer3", ActivationLayer(tf), f"{blk}-2-3x3-norm")
            g.addLayer(f"{blk}-3-pool", SubsamplingLayer(pool, [3, 3], [1, 1], **({"pnorm": 2} if pool == "PNORM" else {"padding": [1, 1]})), src)
            g.addLayer(f"{blk}-3-1x1reduce", _conv((1, 1), nIn=n_in, nOut=96), f"{blk}-3-pool")
            g.addLayer(f"{blk}-3-1x1reduce-norm", BatchNormalization(nIn=96, nOut=96), f"{blk}-3-1x1reduce")
            g.addLayer(f"{blk}-3-transfer4", ActivationLayer("RELU" if blk == "5a" else tf), f"{blk}-3-1x1reduce-norm")
            g.addVertex(f"inception-{blk}", MergeVertex(), f"{blk}-transfer1", f"{blk}-2-transfer3", f"{blk}-3-transfer4")
        g.addLayer("avgpool", _pool("AVG", (3, 3), (3, 3)), "inception-5b")
        g.addLayer("bottleneck", DenseLayer(nOut=self.embeddingSize, activation="IDENTITY"), "avgpool")
        g.addVertex("embeddings", L2NormalizeVertex(None, 1e-6), "bottleneck")
        g.addLayer("lossLayer", CenterLossOutputLayer("SQUARED_LOSS", activation="SOFTMAX", nOut=self.numClasses, lambda_=1e-4, alpha=0.9,
                                                     gradientNormalization=GradientNormalization.RenormalizeL2PerLayer), "embeddings")
        return g.setOutputs("lossLayer").validateOutputLayerConfig(False).build()


# ----------------------------------------------------------------------------- NASNet
class NASNet(ZooModel):
    """NASNet-A (``NASNet.java`` + ``NASNetHelper.java``): stem, three stacks of ``numBlocks`` normal cells separated by
    reduction cells; filters = penultimateFilters / 24."""
    DEFAULT_INPUT = (3, 224, 224)
    DEFAULT_WEIGHT_INIT = "RELU"

    def __init__(self, numBlocks=6, penultimateFilters=1056, stemFilters=96, filterMultiplier=2, skipReduction=True, **kw):
        super().__init__(**kw)
        if penultimateFilters % 24 != 0:
            raise ValueError(f"For NASNet-A models penultimate filters must be divisible by 24. Current value is {penultimateFilters}")
        self.numBlocks, self.penultimateFilters, self.stemFilters = numBlocks, penultimateFilters, stemFilters
        self.filterMultiplier, self.skipReduction = filterMultiplier, skipReduction

    def default_updater(self): return AdaDelta()

    @staticmethod
    def _nbn(): return BatchNormalization(eps=1e-3, gamma=0.9997)

    def _sep_block(self, g, filters, k, stride, block_id, inp):
        p = f"sepConvBlock{block_id}"
        g.addLayer(p + "_act", ActivationLayer("RELU"), inp)
        g.addLayer(p + "_sepconv1", SeparableConvolution2D([k, k], [stride, stride], nOut=filters, hasBias=False, convolutionMode=Same), p + "_act")
        g.addLayer(p + "_conv1_bn", self._nbn(), p + "_sepconv1").addLayer(p + "_act2", ActivationLayer("RELU"), p + "_conv1_bn")
        g.addLayer(p + "_sepconv2", SeparableConvolution2D([k, k], [1, 1], nOut=filters, hasBias=False, convolutionMode=Same), p + "_act2")
        g.addLayer(p + "_conv2_bn", self._nbn(), p + "_sepconv2")
        return p + "_conv2_bn"

    def _adjust(self, g, filters, block_id, inp, to_match=None):
        p = f"adjustBlock{block_id}"
        out = inp
        types = g.getLayerActivationTypes()
        tm, ti = types[to_match or inp], types[inp]
        if tm.height != ti.height:
            g.addLayer(p + "_relu1", ActivationLayer("RELU"), inp)
            g.addLayer(p + "_avgpool1", _pool("AVG", (1, 1), (2, 2), convolutionMode=Truncate), p + "_relu1")
            g.addLayer(p + "_conv1", _conv((1, 1), nOut=filters // 2, hasBias=False, convolutionMode=Same), p + "_avgpool1")
            g.addLayer(p + "_zeropad1", ZeroPaddingLayer(0, 1, 0, 1), p + "_relu1").addLayer(p + "_crop1", Cropping2D(1, 0, 1, 0), p + "_zeropad1")
            g.addLayer(p + "_avgpool2", _pool("AVG", (1, 1), (2, 2), convolutionMode=Truncate), p + "_crop1")
            g.addLayer(p + "_conv2", _conv((1, 1), nOut=filters - filters // 2, hasBias=False, convolutionMode=Same), p + "_avgpool2")
            g.addVertex(p + "_concat1", MergeVertex(), p + "_conv1", p + "_conv2").addLayer(p + "_bn1", self._nbn(), p + "_concat1")
            out = p + "_bn1"
            ti = g.getLayerActivationTypes()[out]
        if ti.channels != filters:
            g.addLayer(p + "_projection_relu", ActivationLayer("RELU"), out)
            g.addLayer(p + "_projection_conv", _conv((1, 1), nOut=filters, hasBias=False, convolutionMode=Same), p + "_projection_relu")
            g.addLayer(p + "_projection_bn", self._nbn(), p + "_projection_conv")
            out = p + "_projection_bn"
        return out

    def _cell_head(self, g, filters, p, x, prev):
        top = self._adjust(g, filters, p, prev if prev is not None else x, x)
        g.addLayer(p + "_relu1", ActivationLayer("RELU"), x).addLayer(p + "_conv1", _conv((1, 1), nOut=filters, hasBias=False, convolutionMode=Same), p + "_relu1")
        g.addLayer(p + "_bn1", self._nbn(), p + "_conv1")
        return top

    def _normal(self, g, filters, block_id, x, prev):
        p = f"normalA{block_id}"
        top = self._cell_head(g, filters, p, x, prev)
        h = p + "_bn1"
        add = lambda n, a, b: g.addVertex(f"{p}_add{n}", ElementWiseVertex("Add"), a, b)
        add(1, self._sep_block(g, filters, 5, 1, p + "_left1", h), self._sep_block(g, filters, 3, 1, p + "_right1", top))
        add(2, self._sep_block(g, filters, 5, 1, p + "_left2", top), self._sep_block(g, filters, 3, 1, p + "_right2", top))
        g.addLayer(p + "_left3", _pool("AVG", (3, 3), (1, 1), convolutionMode=Same), h)
        add(3, p + "_left3", top)
        g.addLayer(p + "_left4", _pool("AVG", (3, 3), (1, 1), convolutionMode=Same), top).addLayer(p + "_right4", _pool("AVG", (3, 3), (1, 1), convolutionMode=Same), top)
        add(4, p + "_left4", p + "_right4")
        add(5, self._sep_block(g, filters, 3, 1, p + "_left5", h), h)
        g.addVertex(p, MergeVertex(), top, *[f"{p}_add{i}" for i in range(1, 6)])
        return p, x

    def _reduction(self, g, filters, block_id, x, prev):
        p = f"reductionA{block_id}"
        top = self._cell_head(g, filters, p, x, prev)
        h = p + "_bn1"
        add = lambda n, a, b: g.addVertex(f"{p}_add{n}", ElementWiseVertex("Add"), a, b)
        add(1, self._sep_block(g, filters, 5, 2, p + "_left1", h), self._sep_block(g, filters, 7, 2, p + "_right1", top))
        g.addLayer(p + "_left2", _pool("MAX", (3, 3), (2, 2), convolutionMode=Same), h)
        add(2, p + "_left2", self._sep_block(g, filters, 7, 2, p + "_right2", top))
        g.addLayer(p + "_left3", _pool("AVG", (3, 3), (2, 2), convolutionMode=Same), h)
        add(3, p + "_left3", self._sep_block(g, filters, 5, 2, p + "_right3", top))
        g.addLayer(p + "_left4", _pool("AVG", (3, 3), (1, 1), convolutionMode=Same), p + "_add1")
        add(4, p + "_add2", p + "_left4")
        g.addLayer(p + "_right5", _pool("MAX", (3, 3), (2, 2), convolutionMode=Same), h)
        add(5, self._sep_block(g, filters, 3, 1, p + "_left5", p + "_add1"), p + "_right5")
        g.addVertex(p, MergeVertex(), *[f"{p}_add{i}" for i in range(2, 6)])
        return p, x

    def conf(self):
        c, h, w = self.inputShape
        filters, fm, nb = self.penultimateFilters // 24, self.filterMultiplier, self.numBlocks
        g = self._base().l2(5e-5).convolutionMode(Truncate).graphBuilder().addInputs("input").setInputTypes(InputType.convolutional(h, w, c))
        g.addLayer("stem_conv1", _conv((3, 3), (1, 1) if self.skipReduction else (2, 2), nOut=self.stemFilters, hasBias=False), "input")
        g.addLayer("stem_bn1", self._nbn(), "stem_conv1")
        x, prev = "stem_bn1", None
        if not self.skipReduction:
            x, prev = self._reduction(g, int(self.stemFilters / fm ** 2), "stem1", "stem_bn1", None)
            x, prev = self._reduction(g, int(self.stemFilters / fm), "stem2", x, prev)
        for stage, mult in enumerate((1, fm, fm ** 2)):
            if stage > 0:
                x, p0 = self._reduction(g, filters * mult, f"reduce{stage * nb}", x, prev)
                prev = p0 if not self.skipReduction else prev
            for i in range(nb):
                x, prev = self._normal(g, filters * mult, str(i + stage * nb + (1 if stage else 0)), x, prev)
        g.addLayer("act", ActivationLayer("RELU"), x).addLayer("avg_pool", GlobalPoolingLayer("AVG"), "act")
        g.addLayer("output", OutputLayer("MCXENT", nOut=self.numClasses, activation="SOFTMAX"), "avg_pool")
        return g.setOutputs("output").build()


ALL_MODELS = {c.__name__: c for c in (LeNet, SimpleCNN, AlexNet, VGG16, VGG19, Darknet19, TinyYOLO, YOLO2, SqueezeNet, UNet, Xception,
                                      InceptionResNetV1, FaceNetNN4Small2, NASNet)}
