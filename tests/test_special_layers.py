"""VAE, locally connected, capsule, YOLOv2, one-class and SameDiff-defined layers on CPU."""
import torch

from deeplearning4j_b200 import nn
from deeplearning4j_b200.data.dataset import DataSet
from deeplearning4j_b200.data.iterators import ListDataSetIterator
from deeplearning4j_b200.nn.conf.neuralnet import MultiLayerConfiguration


def _mln(*layers, input_type=None, updater=None):
    lb = nn.NeuralNetConfiguration.Builder().seed(5).updater(updater or nn.Adam(1e-2)).weightInit("XAVIER").list()
    for l in layers:
        lb.layer(l)
    if input_type is not None:
        lb.setInputType(input_type)
    return nn.MultiLayerNetwork(lb.build()).init()


def test_vae_pretrain_reduces_elbo_and_json_round_trip():
    g = torch.Generator().manual_seed(0)
    x = (torch.rand(64, 12, generator=g) > 0.5).float()
    vae = nn.VariationalAutoencoder(nIn=12, nOut=3, encoderLayerSizes=[16], decoderLayerSizes=[16], activation="tanh",
                                    reconstructionDistribution=nn.BernoulliReconstructionDistribution("sigmoid"), numSamples=2)
    net = _mln(vae, nn.OutputLayer("MSE", nIn=3, nOut=2, activation="identity"))
    conf2 = MultiLayerConfiguration.fromJson(net.conf.toJson())
    assert conf2.toJson() == net.conf.toJson()
    layer = net.conf.layers()[0]
    names = [s.name for s in layer.param_specs()]
    assert names == ["e0W", "e0b", "pZXMeanW", "pZXMeanb", "pZXLogStd2W", "pZXLogStd2b", "d0W", "d0b", "pXZW", "pXZb"]
    it = ListDataSetIterator([DataSet(x, torch.zeros(64, 2))])
    p = net.param_views["0"]
    torch.manual_seed(0)
    before = float(sum(layer.pretrain_score(p, x) for _ in range(8)) / 8)
    net.pretrainLayer(0, it, 60)
    torch.manual_seed(0)
    after = float(sum(layer.pretrain_score(p, x) for _ in range(8)) / 8)
    assert after < before - 0.3
    lp = layer.reconstructionLogProbability(p, x, 4)
    assert lp.shape == (64,) and layer.generateAtMeanGivenZ(p, torch.zeros(5, 3)).shape == (5, 12)
    comp = (nn.CompositeReconstructionDistribution.Builder().addDistribution(4, nn.GaussianReconstructionDistribution())
            .addDistribution(8, nn.BernoulliReconstructionDistribution()).build())
    assert comp.distributionInputSize(12) == 16
    assert comp.exampleNegLogProbability(x, torch.zeros(64, 16)).shape == (64,)


def test_locally_connected_layers_train():
    net = _mln(nn.LocallyConnected2D(nOut=4, kernel=(3, 3), stride=(1, 1), convolutionMode="Truncate", activation="relu"),
               nn.OutputLayer("MCXENT", nOut=3, activation="softmax"), input_type=nn.InputType.convolutional(6, 6, 2))
    assert tuple(net.paramTable()["0_W"].t.shape) == (16, 18, 4)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(16, 2, 6, 6, generator=g)
    y = torch.nn.functional.one_hot(torch.randint(0, 3, (16,), generator=g), 3).float()
    s0 = net.score(DataSet(x, y))
    for _ in range(30):
        net.fit(x, y)
    assert net.score(DataSet(x, y)) < s0
    # untied weights: equals a per-position dense map
    l = net.conf.layers()[0]
    W = net.paramTable()["0_W"].t
    out = l.forward({"W": W, "b": net.paramTable()["0_b"].t}, x, False)
    patch = x[:, :, 1:4, 2:5].reshape(16, -1)
    ref = torch.relu(patch @ W[1 * 4 + 2] + net.paramTable()["0_b"].t)
    assert torch.allclose(out[:, :, 1, 2], ref, atol=1e-5)
    net1 = _mln(nn.LocallyConnected1D(nOut=5, kernel=3, convolutionMode="Same", activation="tanh"), nn.RnnOutputLayer("MSE", nOut=2, activation="identity"),
                input_type=nn.InputType.recurrent(3, 7))
    assert tuple(net1.output(torch.randn(2, 3, 7)).t.shape) == (2, 2, 7)


def test_capsule_network_shapes_and_training():
    net = _mln(nn.ConvolutionLayer([3, 3], nOut=8, activation="relu"),
               nn.PrimaryCapsules(4, 2, kernelSize=(3, 3), stride=(2, 2)),
               nn.CapsuleLayer(3, 6, 2), nn.CapsuleStrengthLayer(),
               nn.LossLayer("MCXENT", activation="softmax"),
               input_type=nn.InputType.convolutional(10, 10, 1))
    g = torch.Generator().manual_seed(2)
    x = torch.randn(8, 1, 10, 10, generator=g)
    y = torch.nn.functional.one_hot(torch.randint(0, 3, (8,), generator=g), 3).float()
    acts = net.feedForward(x)
    acts = [a.t if hasattr(a, 't') and not isinstance(a, torch.Tensor) else a for a in acts]
    assert tuple(acts[2].shape) == (8, 2 * 3 * 3, 4) and tuple(acts[3].shape) == (8, 3, 6) and tuple(acts[4].shape) == (8, 3)
    assert float((acts[3] ** 2).sum(-1).max()) < 1.0                                  # squash keeps capsule norms below 1
    s0 = net.score(DataSet(x, y))
    for _ in range(25):
        net.fit(x, y)
    assert net.score(DataSet(x, y)) < s0


def test_yolo2_output_layer_loss_decreases():
    priors = [[1.0, 1.0], [2.0, 1.5]]
    net = _mln(nn.ConvolutionLayer([1, 1], nOut=2 * (5 + 3), activation="identity"),
               nn.Yolo2OutputLayer(boundingBoxes=priors), input_type=nn.InputType.convolutional(4, 4, 6))
    g = torch.Generator().manual_seed(3)
    x = torch.randn(4, 6, 4, 4, generator=g)
    labels = torch.zeros(4, 4 + 3, 4, 4)
    for n in range(4):
        cy, cx, c = n % 4, (n + 1) % 4, n % 3
        labels[n, 0:4, cy, cx] = torch.tensor([cx + 0.1, cy + 0.2, cx + 0.9, cy + 0.8])
        labels[n, 4 + c, cy, cx] = 1.0
    s0 = net.score(DataSet(x, labels))
    for _ in range(60):
        net.fit(x, labels)
    assert net.score(DataSet(x, labels)) < 0.6 * s0
    out = net.output(x)
    dets = net.conf.layers()[1].getPredictedObjects(out, 0.3)
    assert tuple(out.t.shape) == (4, 16, 4, 4) and isinstance(dets, list)
    assert "boundingBoxes" in net.conf.toJson()


def test_ocnn_output_layer_trains_and_tracks_r():
    net = _mln(nn.DenseLayer(nIn=5, nOut=8, activation="relu"), nn.OCNNOutputLayer(nIn=8, hiddenSize=6, nu=0.1, activation="sigmoid"),
               updater=nn.Adam(1e-2))
    x = torch.randn(64, 5, generator=torch.Generator().manual_seed(4)) * 0.1 + 1.0
    y = torch.zeros(64, 1)
    s0 = net.score(DataSet(x, y))
    for _ in range(40):
        net.fit(x, y)
    assert net.score(DataSet(x, y)) < s0
    r = float(net.paramTable()["1_R"].t)
    scores = net.output(x).t.reshape(-1)
    assert abs(float((scores < r).float().mean()) - 0.1) < 0.08


class _MyDense(nn.SameDiffLayer):
    DEFAULTS = {"nIn": 0, "nOut": 0}

    def defineParameters(self, params):
        params.addWeightParam("W", self.nIn, self.nOut)
        params.addBiasParam("b", 1, self.nOut)

    def defineLayer(self, sd, layerInput, paramTable, mask=None):
        return sd.nn.tanh(layerInput.mmul(paramTable["W"]).add(paramTable["b"]))

    def getOutputType(self, idx, it):
        return nn.InputType.feedForward(self.nOut)


class _Scale(nn.SameDiffLambdaLayer):
    def defineLayer(self, sd, layerInput):
        return layerInput.mul(2.0)


def test_samediff_defined_layers_match_dense_and_train():
    net = _mln(_MyDense(nIn=4, nOut=6), _Scale(), nn.OutputLayer("MSE", nIn=6, nOut=2, activation="identity"))
    x = torch.randn(10, 4, generator=torch.Generator().manual_seed(6))
    W, b = net.paramTable()["0_W"].t, net.paramTable()["0_b"].t
    a2 = net.feedForward(x)[2]
    a2 = a2 if isinstance(a2, torch.Tensor) else a2.t
    assert torch.allclose(a2, 2 * torch.tanh(x @ W + b), atol=1e-6)
    y = torch.randn(10, 2, generator=torch.Generator().manual_seed(7))
    s0 = net.score(DataSet(x, y))
    for _ in range(30):
        net.fit(x, y)
    assert net.score(DataSet(x, y)) < s0


def test_stride2_stem_space_to_depth_rewrite_is_exact():
    """The RGB-stem rewrite used on the GPU path (stride-2 conv -> stride-1 conv over a 2x2 space-to-depth view)."""
    import torch.nn.functional as F
    from deeplearning4j_b200.nn.layers.conv import _stem_space_to_depth
    g = torch.Generator().manual_seed(0)
    for (H, W, k, p) in [(64, 64, (7, 7), (3, 3)), (33, 31, (3, 3), (1, 1)), (32, 32, (5, 3), (2, 0)), (17, 18, (2, 2), (0, 0))]:
        x = torch.randn(2, 3, H, W, dtype=torch.float64, generator=g)
        w = torch.randn(5, 3, *k, dtype=torch.float64, generator=g)
        b = torch.randn(5, dtype=torch.float64, generator=g)
        ref = F.conv2d(x, w, b, stride=2, padding=p)
        got = _stem_space_to_depth(x, w, b, k, p)
        assert got.shape == ref.shape and float((got - ref).abs().max()) < 1e-10
