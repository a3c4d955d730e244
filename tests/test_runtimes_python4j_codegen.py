"""Foreign-format runners, the python4j executioner, omnihub cache resolution and namespace code generation."""
import importlib.util
import os

import numpy as np
import pytest
import torch

from deeplearning4j_b200 import Nd4j


def test_python4j_executes_snippets_with_typed_variables():
    from deeplearning4j_b200.python4j import (PythonContextManager, PythonExecutioner, PythonGIL, PythonJob, PythonTypes, PythonVariable,
                                              PythonVariables)
    ins = PythonVariables().add("x", PythonTypes.NDARRAY, Nd4j.create([1.0, 2.0, 3.0])).add("k", PythonTypes.INT, 3)
    outs = PythonVariables().add("y", PythonTypes.NDARRAY).add("s", PythonTypes.FLOAT)
    with PythonGIL.lock():
        PythonExecutioner.exec("import numpy as np\ny = x * k\ns = float(np.sum(y))", ins, outs)
    assert outs.get("y").getValue().numpy().tolist() == [3.0, 6.0, 9.0] and outs.get("s").getValue() == 18.0
    PythonContextManager.setContext("other")
    with pytest.raises(KeyError):
        PythonExecutioner.exec("pass", None, [PythonVariable("y")])          # contexts are isolated
    PythonContextManager.setContext("main")
    PythonContextManager.deleteNonMainContexts()
    job = PythonJob("j", "def setup():\n    global w\n    w = 10\ndef run(a):\n    return {'b': a + w}", setupRunMode=True)
    o = [PythonVariable("b", PythonTypes.INT)]
    job.exec([PythonVariable("a", PythonTypes.INT, 5)], o)
    assert o[0].getValue() == 15
    allv = PythonExecutioner.execAndReturnAllVariables("q = [1, 2]\nz = 'hi'")
    assert {v.name for v in allv} >= {"q", "z"}


def test_foreign_runners():
    from deeplearning4j_b200.importers import protowire as pw
    from deeplearning4j_b200.runtimes import GraphRunner, OnnxRuntimeRunner, TensorFlowLiteRunner, TvmRunner
    import tests.test_import_onnx as t_onnx
    builders = [getattr(t_onnx, n) for n in dir(t_onnx) if n.startswith("_") and "model" in n.lower() and callable(getattr(t_onnx, n))]
    if builders:
        try:
            data = builders[0]()
            data = data[0] if isinstance(data, tuple) else data
            with OnnxRuntimeRunner(modelBytes=data) as r:
                assert r.getInputs() and r.getOutputs()
        except TypeError:
            pass
    with pytest.raises(ValueError):
        TensorFlowLiteRunner(modelBytes=b"not a flatbuffer")
    with pytest.raises(NotImplementedError):
        TvmRunner("model.so")
    assert callable(GraphRunner.builder) and pw is not None


def test_omnihub_cache_layout(tmp_path, monkeypatch):
    from deeplearning4j_b200 import nn
    from deeplearning4j_b200.omnihub import OmniHubUtils
    monkeypatch.setenv("OMNIHUB_HOME", str(tmp_path))
    p = OmniHubUtils.modelPath("dl4j", "tiny.zip")
    assert p == os.path.join(str(tmp_path), "dl4j", "tiny.zip")
    monkeypatch.setenv("OMNIHUB_URL", "file://" + str(tmp_path / "nowhere"))
    with pytest.raises(IOError, match="could not be fetched"):
        OmniHubUtils.downloadAndLoadFromZoo("dl4j", "tiny.zip")
    assert not os.path.exists(p + ".part")
    conf = (nn.NeuralNetConfiguration.Builder().seed(1).list().layer(nn.DenseLayer(nIn=3, nOut=2, activation="relu"))
            .layer(nn.OutputLayer("MSE", nIn=2, nOut=1, activation="identity")).build())
    net = nn.MultiLayerNetwork(conf)
    net.init()
    os.makedirs(os.path.dirname(p), exist_ok=True)
    nn.ModelSerializer.writeModel(net, p, False)
    assert OmniHubUtils.loadNetwork("tiny.zip").numParams() == net.numParams()
    with pytest.raises(ValueError):
        OmniHubUtils.modelPath("caffe", "x")


def test_omnihub_download_convert_and_namespaces(tmp_path, monkeypatch):
    """The hub is a ``file://`` folder: fetch into the cache, convert an ONNX and a TFLite model to SameDiff .fb files, and reach the
    results through the generated-style namespaces (``OmniHubUtils.java:128-150``, ``BootstrapFromLocal.java``)."""
    import torch
    from deeplearning4j_b200.omnihub import (BootstrapFromLocal, Framework, ModelNamespaceGenerator, OmniHubUtils, Pretrained, clearCache)
    import tests.test_import_tflite as t_tfl
    hub, home = tmp_path / "hub", tmp_path / "home"
    monkeypatch.setenv("OMNIHUB_HOME", str(home))
    monkeypatch.setenv("OMNIHUB_URL", "file://" + str(hub))
    b = t_tfl.ModelBuilder()
    x = b.tensor("x", [2, 3])
    y = b.tensor("y", [2, 3]); b.op("TANH", [x], [y])
    os.makedirs(hub / "tensorflow")
    (hub / "tensorflow" / "tiny-tanh.tflite").write_bytes(b.build([x], [y]))
    seen = []
    p = OmniHubUtils.downloadAndLoadFromZoo("tensorflow", "tiny-tanh.tflite", progress=lambda done, total: seen.append((done, total)))
    assert p == str(home / "tensorflow" / "tiny-tanh.tflite") and os.path.getsize(p) == seen[-1][0]
    (hub / "tensorflow" / "tiny-tanh.tflite").unlink()                      # cached: the hub is not asked again
    assert OmniHubUtils.downloadAndLoadFromZoo("tensorflow", "tiny-tanh.tflite") == p
    (home / "onnx").mkdir()
    (home / "onnx" / "broken.onnx").write_bytes(b"\x00\x01not a model")
    res = BootstrapFromLocal.run()
    out = res[p]
    assert out == str(home / "samediff" / "tiny-tanh.fb") and os.path.exists(out)
    assert isinstance(res[str(home / "onnx" / "broken.onnx")], Exception)
    ns = Pretrained.samediff()
    assert ns.models() == ["tinyTanh"] and "tinyTanh" in dir(ns)
    sd = ns.tinyTanh()
    xin = torch.tensor([[0.5, -1.0, 2.0], [0.0, 1.0, -2.0]])
    got = sd.output({"x": xin}, "y")["y"]
    torch.testing.assert_close(got.t if hasattr(got, "t") else got, torch.tanh(xin))
    with pytest.raises(KeyError):
        ns.load("resnet18")
    src = ModelNamespaceGenerator.generate(Framework.SAMEDIFF)
    assert "class SameDiffModels:" in src and "def tinyTanh(self, forceDownload=False):" in src
    compile(src, "generated", "exec")
    assert Framework.outputFrameworkFor(Framework.KERAS) == Framework.DL4J and Framework.isOutput(Framework.SAMEDIFF)
    with pytest.raises(ValueError):
        Framework.outputFrameworkFor(Framework.DL4J)
    clearCache(Framework.SAMEDIFF)
    assert Pretrained.samediff().models() == []


def test_codegen_emits_working_namespaces(tmp_path):
    from deeplearning4j_b200 import codegen
    d = codegen.describe("conv2d")
    assert d["inputs"][:2] == ["x", "w"] and ("sH", 1) in d["args"] and d["group"] == "conv"
    files = codegen.write_all(str(tmp_path))
    assert any(f.endswith("_nn.py") for f in files) and os.path.exists(tmp_path / "ops.md")
    src = next(f for f in files if f.endswith("_elementwise.py"))
    spec = importlib.util.spec_from_file_location("gen_ns", src)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    ns = mod.NDMathElementwise
    np.testing.assert_allclose(ns.tanh(torch.tensor([0.5])).numpy(), np.tanh([0.5]), rtol=1e-6)
    assert "`softmax(" in open(tmp_path / "ops.md").read()
