"""NVTX ranges (utils/nvtx.py): per layer, per updater step and per SameDiff op, balanced, and absent when switched off."""
import torch

from deeplearning4j_b200 import nn
from deeplearning4j_b200.data import DataSet
from deeplearning4j_b200.utils import nvtx


def _net():
    conf = (nn.NeuralNetConfiguration.Builder().seed(1).updater(nn.Sgd(0.1)).list()
            .layer(nn.DenseLayer(nIn=4, nOut=3, activation="tanh"))
            .layer(nn.OutputLayer("MSE", nIn=3, nOut=2, activation="identity")).build())
    return nn.MultiLayerNetwork(conf).init()


def test_ranges_per_layer_and_updater_and_off_by_default():
    net, log = _net(), []
    ds = DataSet(torch.rand(5, 4), torch.rand(5, 2))
    nvtx.record(log)
    try:
        net.fit(ds)
        assert log == []                                   # disabled: nothing is pushed
        nvtx.enable(True)
        net.fit(ds)
    finally:
        nvtx.enable(False)
        nvtx.record(None)
    names = [n for e, n in log if e == "push"]
    assert "layer 0 DenseLayer" in names and "layer 1 OutputLayer" in names and "updater" in names
    depth = 0
    for e, _ in log:
        depth += 1 if e == "push" else -1
        assert depth >= 0
    assert depth == 0


def test_samediff_listener_ranges():
    from deeplearning4j_b200.samediff import SameDiff
    sd = SameDiff.create()
    x = sd.placeHolder("x", None, 2, 3)
    y = sd.math.tanh(x).add(1.0)
    log = []
    nvtx.record(log)
    try:
        sd.setListeners(nvtx.NvtxListener())
        sd.output({"x": torch.zeros(2, 3)}, y.name)
    finally:
        nvtx.record(None)
    pushes = [n for e, n in log if e == "push"]
    assert any(n.startswith("tanh:") for n in pushes) and len(pushes) == sum(1 for e, _ in log if e == "pop")
