"""Central-difference gradient checks of layer implementations (the reference's GradientCheckTests* suites)."""
import pytest
import torch

from deeplearning4j_b200 import nn
from deeplearning4j_b200.nn.gradientcheck import GradientCheckUtil


def _check(layers, x, y, input_type=None, **kw):
    lb = nn.NeuralNetConfiguration.Builder().seed(12345).updater(nn.NoOp()).weightInit("XAVIER").list()
    for l in layers:
        lb.layer(l)
    if input_type is not None:
        lb.setInputType(input_type)
    net = nn.MultiLayerNetwork(lb.build()).init()
    ok, fails, checked = GradientCheckUtil.checkGradients(net, x, y, returnDetails=True, subset=True, maxPerParam=25, **kw)
    assert ok and checked > 0, fails[:5]


def _cls(n, c, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.nn.functional.one_hot(torch.randint(0, c, (n,), generator=g), c).double()


def test_dense_activations_and_losses():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(6, 5, generator=g)
    for act in ("tanh", "sigmoid", "softplus", "elu", "gelu", "swish", "cube"):
        _check([nn.DenseLayer(nIn=5, nOut=7, activation=act), nn.OutputLayer("MCXENT", nIn=7, nOut=3, activation="softmax")], x, _cls(6, 3))
    for loss, act in (("MSE", "identity"), ("L2", "tanh"), ("MEAN_ABSOLUTE_ERROR", "identity"), ("XENT", "sigmoid"), ("KL_DIVERGENCE", "softmax"), ("HINGE", "identity"),
                      ("COSINE_PROXIMITY", "identity"), ("POISSON", "softplus")):
        y = torch.rand(6, 3, generator=g).double() + 0.1
        if loss in ("KL_DIVERGENCE",):
            y = y / y.sum(1, keepdim=True)
        if loss == "HINGE":
            y = _cls(6, 3) * 2 - 1
        if loss == "XENT":
            y = (y > 0.5).double()
        _check([nn.DenseLayer(nIn=5, nOut=4, activation="tanh"), nn.OutputLayer(loss, nIn=4, nOut=3, activation=act)], x, y)


def test_cnn_stack_batchnorm_pooling():
    g = torch.Generator().manual_seed(2)
    x = torch.randn(4, 2, 8, 8, generator=g)
    _check([nn.ConvolutionLayer([3, 3], nOut=3, activation="tanh"), nn.BatchNormalization(), nn.SubsamplingLayer("MAX", [2, 2], [2, 2]),
            nn.ConvolutionLayer([2, 2], [1, 1], [1, 1], nOut=2, activation="sigmoid", convolutionMode="Truncate"), nn.SubsamplingLayer("AVG", [2, 2], [1, 1]),
            nn.OutputLayer("MCXENT", nOut=3, activation="softmax")], x, _cls(4, 3), nn.InputType.convolutional(8, 8, 2), maxRelError=1e-2)
    _check([nn.SeparableConvolution2D([3, 3], nOut=4, activation="tanh", convolutionMode="Same"), nn.DepthwiseConvolution2D([2, 2], depthMultiplier=2, activation="tanh"),
            nn.Deconvolution2D([2, 2], [2, 2], nOut=2, activation="tanh"), nn.GlobalPoolingLayer("PNORM"), nn.OutputLayer("MSE", nOut=2, activation="identity")],
           x, torch.randn(4, 2, generator=g).double(), nn.InputType.convolutional(8, 8, 2), maxRelError=1e-2)


def test_recurrent_layers_with_masks():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(3, 4, 6, generator=g)
    y = torch.nn.functional.one_hot(torch.randint(0, 3, (3, 6), generator=g), 3).permute(0, 2, 1).double()
    mask = torch.tensor([[1.0, 1, 1, 1, 1, 1], [1, 1, 1, 1, 0, 0], [1, 1, 0, 0, 0, 0]])
    for rnn in (nn.LSTM(nIn=4, nOut=5, activation="tanh"), nn.GravesLSTM(nIn=4, nOut=5, activation="tanh"), nn.SimpleRnn(nIn=4, nOut=5, activation="tanh"),
                nn.Bidirectional(nn.LSTM(nIn=4, nOut=5, activation="tanh"), mode="CONCAT")):
        n_out = 10 if isinstance(rnn, nn.Bidirectional) else 5
        _check([rnn, nn.RnnOutputLayer("MCXENT", nIn=n_out, nOut=3, activation="softmax")], x, y, inputMask=mask, labelMask=mask)


def test_attention_embedding_and_special_layers():
    g = torch.Generator().manual_seed(4)
    x = torch.randn(3, 4, 5, generator=g)
    y = _cls(3, 2)
    _check([nn.SelfAttentionLayer(nIn=4, nOut=6, nHeads=2, headSize=3, projectInput=True), nn.GlobalPoolingLayer("AVG"),
            nn.OutputLayer("MCXENT", nIn=6, nOut=2, activation="softmax")], x, y, maxRelError=1e-2)
    _check([nn.LearnedSelfAttentionLayer(nIn=4, nOut=6, nHeads=1, headSize=6, nQueries=2, projectInput=True), nn.GlobalPoolingLayer("MAX"),
            nn.OutputLayer("MCXENT", nIn=6, nOut=2, activation="softmax")], x, y, maxRelError=1e-2)
    idx = torch.randint(0, 7, (5, 1), generator=g).float()
    _check([nn.EmbeddingLayer(nIn=7, nOut=4, activation="tanh"), nn.OutputLayer("MCXENT", nIn=4, nOut=3, activation="softmax")], idx, _cls(5, 3))
    _check([nn.LocallyConnected2D(nOut=2, kernel=(2, 2), convolutionMode="Truncate", activation="tanh"), nn.OutputLayer("MSE", nOut=2, activation="identity")],
           torch.randn(3, 1, 4, 4, generator=g), torch.randn(3, 2, generator=g).double(), nn.InputType.convolutional(4, 4, 1))
    _check([nn.PrimaryCapsules(4, 2, kernelSize=(2, 2), stride=(1, 1)), nn.CapsuleLayer(2, 3, 2), nn.CapsuleStrengthLayer(), nn.LossLayer("MSE", activation="identity")],
           torch.randn(2, 1, 4, 4, generator=g), torch.rand(2, 2, generator=g).double(), nn.InputType.convolutional(4, 4, 1), maxRelError=1e-2)
