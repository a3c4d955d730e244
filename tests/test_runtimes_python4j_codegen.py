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
    with pytest.raises(IOError, match="cannot be downloaded"):
        OmniHubUtils.downloadAndLoadFromZoo("dl4j", "tiny.zip")
    conf = (nn.NeuralNetConfiguration.Builder().seed(1).list().layer(nn.DenseLayer(nIn=3, nOut=2, activation="relu"))
            .layer(nn.OutputLayer("MSE", nIn=2, nOut=1, activation="identity")).build())
    net = nn.MultiLayerNetwork(conf)
    net.init()
    os.makedirs(os.path.dirname(p))
    nn.ModelSerializer.writeModel(net, p, False)
    assert OmniHubUtils.loadNetwork("tiny.zip").numParams() == net.numParams()
    with pytest.raises(ValueError):
        OmniHubUtils.modelPath("caffe", "x")


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
