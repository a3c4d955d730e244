"""Runners for models in foreign formats (``nd4j-onnxruntime`` ``OnnxRuntimeRunner``, ``nd4j-tensorflow`` ``GraphRunner``,
``nd4j-tensorflow-lite`` ``TensorFlowLiteRunner``, ``nd4j-tvm`` ``TvmRunner``).

The reference binds each vendor runtime through JavaCPP and feeds it INDArrays.  None of those runtimes is available here, so the
ONNX and TensorFlow runners execute the model through this framework's own importers (protobuf wire reader -> SameDiff graph ->
native kernels); the API (construct from a path or bytes, ``exec`` / ``run`` a name -> array map, ``close``) is the reference's.
TFLite flatbuffers go through ``importers/tflite_import.py`` the same way.  TVM compiled modules (machine code for another
runtime) have no importer and raise on construction."""
from __future__ import annotations

from ..nd.ndarray import INDArray


def _read(model):
    if isinstance(model, (bytes, bytearray)):
        return bytes(model)
    with open(model, "rb") as f:
        return f.read()


class OnnxRuntimeRunner:
    def __init__(self, modelUri=None, modelBytes=None):
        from ..importers import importOnnx
        self.sd = importOnnx(modelBytes if modelBytes is not None else _read(modelUri), trainable=False)
        self.inputs = [v.name_() for v in self.sd.getVariables() if v.isPlaceHolder()]
        self.outputs = list(self.sd.outputs())

    @staticmethod
    def builder():
        class B:
            def __init__(s): s.kw = {}
            def modelUri(s, u): s.kw["modelUri"] = u; return s
            def modelBytes(s, b): s.kw["modelBytes"] = b; return s
            def build(s): return OnnxRuntimeRunner(**s.kw)
        return B()

    def getInputs(self): return list(self.inputs)
    def getOutputs(self): return list(self.outputs)

    def exec(self, inputs: dict) -> dict:
        res = self.sd.output(inputs, *self.outputs)
        return {k: (v if isinstance(v, INDArray) else INDArray(v)) for k, v in res.items()}

    run = exec

    def close(self):
        self.sd = None

    def __enter__(self): return self
    def __exit__(self, *a): self.close()


class GraphRunner:
    """Frozen TensorFlow ``GraphDef`` runner (``GraphRunner.builder().graphBytes(..).inputNames(..).outputNames(..).build()``)."""

    def __init__(self, graphBytes=None, graphPath=None, inputNames=None, outputNames=None, **_session_config):
        from ..importers import importFrozenTF
        self.sd = importFrozenTF(graphBytes if graphBytes is not None else _read(graphPath))
        self.inputNames = list(inputNames) if inputNames else [v.name_() for v in self.sd.getVariables() if v.isPlaceHolder()]
        self.outputNames = list(outputNames) if outputNames else list(self.sd.outputs())

    @staticmethod
    def builder():
        class B:
            def __init__(s): s.kw = {}
            def __getattr__(s, k):
                def f(v):
                    s.kw[k] = v
                    return s
                return f
            def build(s): return GraphRunner(**s.kw)
        return B()

    def run(self, inputs: dict) -> dict:
        res = self.sd.output(inputs, *self.outputNames)
        return {k: (v if isinstance(v, INDArray) else INDArray(v)) for k, v in res.items()}

    exec = run

    def close(self):
        self.sd = None

    def __enter__(self): return self
    def __exit__(self, *a): self.close()


class _Unavailable:
    RUNTIME = ""

    def __init__(self, *a, **kw):
        raise NotImplementedError(f"{self.RUNTIME} models cannot be executed: no {self.RUNTIME} runtime is bundled and no importer for its "
                                  f"file format exists; convert the model to ONNX or a frozen TensorFlow GraphDef and use "
                                  f"OnnxRuntimeRunner / GraphRunner")


class TensorFlowLiteRunner:
    """``TensorFlowLiteRunner.builder().modelUri(path).build()``; ``exec`` maps input tensor names to arrays and returns the model's
    output tensors by name (``nd4j-tensorflow-lite/.../runner/TensorFlowLiteRunner.java``)."""

    def __init__(self, modelUri=None, modelBytes=None):
        from ..importers.tflite_import import TFLiteImporter
        imp = TFLiteImporter(trainable=False)
        self.sd = imp.runImport(modelBytes if modelBytes is not None else _read(modelUri))
        self.inputs, self.outputs = list(imp.inputs), list(imp.outputs)

    builder = staticmethod(lambda: _UriBuilder(TensorFlowLiteRunner))

    def getInputs(self): return list(self.inputs)
    def getOutputs(self): return list(self.outputs)

    def exec(self, inputs: dict) -> dict:
        res = self.sd.output(inputs, *self.outputs)
        return {k: (v if isinstance(v, INDArray) else INDArray(v)) for k, v in res.items()}

    run = exec

    def close(self):
        self.sd = None

    def __enter__(self): return self
    def __exit__(self, *a): self.close()


class _UriBuilder:
    def __init__(self, cls): self.cls, self.kw = cls, {}
    def modelUri(self, u): self.kw["modelUri"] = u; return self
    def modelBytes(self, b): self.kw["modelBytes"] = b; return self
    def build(self): return self.cls(**self.kw)


class TvmRunner(_Unavailable):
    RUNTIME = "TVM"
