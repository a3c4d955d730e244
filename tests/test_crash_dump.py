"""An out-of-memory error during fit leaves a memory crash dump behind and is re-raised (the error is made on the host)."""
import os

import pytest
import torch

from deeplearning4j_b200 import nn
from deeplearning4j_b200.utils.crash import CrashReportingUtil


def _net():
    conf = (nn.NeuralNetConfiguration.Builder().seed(1).updater(nn.Adam(1e-3)).list()
            .layer(nn.DenseLayer(nIn=4, nOut=8, activation="relu")).layer(nn.OutputLayer("MCXENT", nIn=8, nOut=3, activation="softmax")).build())
    return nn.MultiLayerNetwork(conf).init()


def test_oom_in_fit_writes_a_dump_and_re_raises(tmp_path, monkeypatch):
    net = _net()
    CrashReportingUtil.crashDumpOutputDirectory(str(tmp_path))
    try:
        def boom(*a, **kw):
            raise MemoryError("CUDA out of memory (injected on the host)")
        monkeypatch.setattr(net, "_fit_arrays", boom)
        with pytest.raises(MemoryError, match="memory crash dump written to"):
            net.fit(torch.rand(5, 4), torch.eye(3)[torch.randint(0, 3, (5,))])
        files = [f for f in os.listdir(tmp_path) if f.startswith("dl4j-memory-crash-dump-")]
        assert len(files) == 1
        text = open(os.path.join(tmp_path, files[0])).read()
        assert "Network # Parameters: 67" in text and "Updater state: 134 values" in text and "injected on the host" in text
        assert "========== Layer Information ==========" in text
        # other errors pass through untouched, and dumps can be switched off
        monkeypatch.setattr(net, "_fit_arrays", lambda *a, **kw: (_ for _ in ()).throw(ValueError("bad shape")))
        with pytest.raises(ValueError, match="^bad shape$"):
            net.fit(torch.rand(5, 4), torch.rand(5, 3))
        CrashReportingUtil.crashDumpsEnabled(False)
        monkeypatch.setattr(net, "_fit_arrays", boom)
        with pytest.raises(MemoryError):
            net.fit(torch.rand(5, 4), torch.rand(5, 3))
        assert len([f for f in os.listdir(tmp_path) if f.startswith("dl4j-memory-crash-dump-")]) == 1
    finally:
        CrashReportingUtil.crashDumpsEnabled(True)
        CrashReportingUtil.crashDumpOutputDirectory(None)
