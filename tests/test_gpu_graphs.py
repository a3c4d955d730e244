"""CUDA-graph replay of the training step (setCudaGraphs) must give the same parameters as eager execution, for a
feed-forward network and for truncated BPTT with carried recurrent state."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mlp(graphs):
    from deeplearning4j_b200 import DataType, nn
    conf = (nn.NeuralNetConfiguration.Builder().seed(11).updater(nn.Adam(1e-2)).computeDataType(DataType.BFLOAT16).list()
            .layer(nn.DenseLayer(nIn=64, nOut=128, activation="relu"))
            .layer(nn.DenseLayer(nIn=128, nOut=128, activation="tanh"))
            .layer(nn.OutputLayer("MCXENT", nIn=128, nOut=8, activation="softmax")).build())
    net = nn.MultiLayerNetwork(conf)
    net.device = torch.device("cuda")
    net.init()
    if graphs:
        net.setCudaGraphs(True)
    return net


def test_mlp_graph_replay_matches_eager():
    from deeplearning4j_b200.ops import native
    native.require()
    rng = np.random.default_rng(0)
    batches = [(torch.tensor(rng.normal(size=(32, 64)).astype(np.float32), device="cuda"),
                torch.tensor(np.eye(8, dtype=np.float32)[rng.integers(0, 8, size=32)], device="cuda")) for _ in range(6)]
    a, b = _mlp(True), _mlp(False)
    for x, y in batches:
        a.fit(x, y)
        b.fit(x, y)
    assert any(e["graph"] is not None for e in a._cg["entries"].values())
    pa, pb = a.params().numpy(), b.params().numpy()
    assert np.abs(pa - pb).max() < 2e-3 * (np.abs(pb).max() + 1e-6)
    assert abs(a.score() - b.score()) < 2e-2 * (abs(b.score()) + 1e-6)
    native.check_status()


def _lstm(graphs):
    from deeplearning4j_b200 import DataType, nn
    conf = (nn.NeuralNetConfiguration.Builder().seed(5).updater(nn.Adam(1e-2)).computeDataType(DataType.BFLOAT16).graphBuilder()
            .addInputs("in")
            .addLayer("l1", nn.LSTM(nIn=16, nOut=64, activation="tanh"), "in")
            .addLayer("out", nn.RnnOutputLayer("MCXENT", nIn=64, nOut=16, activation="softmax"), "l1")
            .setOutputs("out").backpropType("TruncatedBPTT").tBPTTForwardLength(8).tBPTTBackwardLength(8).build())
    net = nn.ComputationGraph(conf)
    net.device = torch.device("cuda")
    net.init()
    if graphs:
        net.setCudaGraphs(True)
    return net


def test_tbptt_graph_replay_carries_state_like_eager():
    from deeplearning4j_b200.ops import native
    native.require()
    rng = np.random.default_rng(1)
    idx = rng.integers(0, 16, size=(8, 33))
    x = torch.tensor(np.eye(16, dtype=np.float32)[idx[:, :-1]].transpose(0, 2, 1).copy(), device="cuda")
    y = torch.tensor(np.eye(16, dtype=np.float32)[idx[:, 1:]].transpose(0, 2, 1).copy(), device="cuda")
    a, b = _lstm(True), _lstm(False)
    for _ in range(3):                          # 3 fits x 4 segments: the later ones replay captured graphs
        a.fit(x, y)
        b.fit(x, y)
    assert sum(e["graph"] is not None for e in a._cg["entries"].values()) >= 2      # first segment and state-carrying segments
    pa, pb = a.params().numpy(), b.params().numpy()
    assert np.abs(pa - pb).max() < 5e-3 * (np.abs(pb).max() + 1e-6)
    native.check_status()
