"""``ComputationGraphConfiguration`` (+ ``GraphBuilder``) and the graph vertices
(``deeplearning4j-nn/.../nn/conf/ComputationGraphConfiguration.java``, ``nn/conf/graph/*.java`` and
``nn/conf/graph/rnn/*.java``).  JSON keeps the reference's shape: ``vertices`` (name -> typed vertex),
``vertexInputs`` (name -> input names), ``networkInputs`` / ``networkOutputs``."""
from __future__ import annotations

import torch

from ...nd.dtype import DataType
from ...serde import jackson
from .base import BackpropType, CacheMode, InputType, Layer, RNNFormat, WorkspaceMode
from .neuralnet import NeuralNetConfiguration, _unbuild
from .preprocessors import preprocessor_from_json

_G = "org.deeplearning4j.nn.conf.graph."


class GraphVertex:
    JAVA = ""
    FIELDS: tuple = ()
    HAS_PARAMS = False

    def forward(self, inputs, training, masks=None, ctx=None):
        raise NotImplementedError

    def output_type(self, *its):
        return its[0]

    def param_specs(self):
        return []

    def mask_out(self, masks):
        ms = [m for m in (masks or []) if m is not None]
        return ms[0] if ms else None

    def to_json(self):
        d = {"@class": _G + self.JAVA}
        for f in self.FIELDS:
            v = getattr(self, f)
            d[f] = v.to_json() if hasattr(v, "to_json") else v
        return d

    def __eq__(self, o):
        return type(self) is type(o) and self.to_json() == o.to_json()


class LayerVertex(GraphVertex):
    JAVA = "LayerVertex"

    def __init__(self, layer, preProcessor=None, conf=None):
        self.layer, self.preProcessor = layer, preProcessor
        self.conf = conf or NeuralNetConfiguration(layer)

    @property
    def HAS_PARAMS(self):
        return self.layer.HAS_PARAMS

    def param_specs(self):
        return self.layer.param_specs()

    def output_type(self, *its):
        it = its[0]
        if self.preProcessor is not None:
            it = self.preProcessor.output_type(it)
        return self.layer.output_type(it)

    def to_json(self):
        c = self.conf.to_json()
        return {"@class": _G + self.JAVA, "layerConf": c, "outputVertex": False,
                "preProcessor": self.preProcessor.to_json() if self.preProcessor else None}


class ElementWiseVertex(GraphVertex):
    JAVA = "ElementWiseVertex"; FIELDS = ("op",)

    class Op:
        Add = "Add"; Subtract = "Subtract"; Product = "Product"; Average = "Average"; Max = "Max"

    def __init__(self, op="Add"):
        self.op = op

    def forward(self, inputs, training, masks=None, ctx=None):
        if self.op == "Add":
            y = inputs[0]
            for x in inputs[1:]:
                y = y + x
            return y
        if self.op == "Subtract":
            return inputs[0] - inputs[1]
        if self.op == "Product":
            y = inputs[0]
            for x in inputs[1:]:
                y = y * x
            return y
        if self.op == "Average":
            return torch.stack(inputs).mean(0)
        if self.op == "Max":
            return torch.stack(inputs).amax(0)
        raise ValueError(self.op)


class MergeVertex(GraphVertex):
    JAVA = "MergeVertex"; FIELDS = ("mergeAxis",)

    def __init__(self, mergeAxis=1):
        self.mergeAxis = mergeAxis

    def forward(self, inputs, training, masks=None, ctx=None):
        return inputs[0] if len(inputs) == 1 else torch.cat(inputs, dim=self.mergeAxis)

    def output_type(self, *its):
        a = its[0]
        if a.kind == InputType.FF:
            return InputType.feedForward(sum(i.size for i in its))
        if a.kind == InputType.RNN:
            return InputType.recurrent(sum(i.size for i in its), a.timeSeriesLength, a.format)
        if a.kind == InputType.CNN:
            return InputType.convolutional(a.height, a.width, sum(i.channels for i in its), a.format)
        if a.kind == InputType.CNN3D:
            return InputType.convolutional3D(a.depth, a.height, a.width, sum(i.channels for i in its))
        return a


class SubsetVertex(GraphVertex):
    JAVA = "SubsetVertex"; FIELDS = ("from", "to")

    def __init__(self, frm, to):
        setattr(self, "from", frm)
        self.to = to

    def forward(self, inputs, training, masks=None, ctx=None):
        return inputs[0][:, getattr(self, "from"):self.to + 1]

    def output_type(self, *its):
        n = self.to - getattr(self, "from") + 1
        a = its[0]
        if a.kind == InputType.RNN:
            return InputType.recurrent(n, a.timeSeriesLength, a.format)
        if a.kind == InputType.CNN:
            return InputType.convolutional(a.height, a.width, n, a.format)
        return InputType.feedForward(n)


class StackVertex(GraphVertex):
    JAVA = "StackVertex"

    def forward(self, inputs, training, masks=None, ctx=None):
        return torch.cat(inputs, dim=0)

    def mask_out(self, masks):
        ms = [m for m in (masks or [])]
        return torch.cat(ms, 0) if ms and all(m is not None for m in ms) else None


class UnstackVertex(GraphVertex):
    JAVA = "UnstackVertex"; FIELDS = ("from", "stackSize")

    def __init__(self, frm, stackSize):
        setattr(self, "from", frm)
        self.stackSize = stackSize

    def forward(self, inputs, training, masks=None, ctx=None):
        x = inputs[0]
        step = x.shape[0] // self.stackSize
        f = getattr(self, "from")
        return x[f * step:(f + 1) * step]

    def mask_out(self, masks):
        m = masks[0] if masks else None
        if m is None:
            return None
        step = m.shape[0] // self.stackSize
        f = getattr(self, "from")
        return m[f * step:(f + 1) * step]


class ScaleVertex(GraphVertex):
    JAVA = "ScaleVertex"; FIELDS = ("scaleFactor",)
    def __init__(self, scaleFactor=1.0): self.scaleFactor = float(scaleFactor)
    def forward(self, inputs, training, masks=None, ctx=None): return inputs[0] * self.scaleFactor


class ShiftVertex(GraphVertex):
    JAVA = "ShiftVertex"; FIELDS = ("shiftFactor",)
    def __init__(self, shiftFactor=0.0): self.shiftFactor = float(shiftFactor)
    def forward(self, inputs, training, masks=None, ctx=None): return inputs[0] + self.shiftFactor


class L2NormalizeVertex(GraphVertex):
    JAVA = "L2NormalizeVertex"; FIELDS = ("dimension", "eps")
    def __init__(self, dimension=None, eps=1e-8): self.dimension, self.eps = dimension, eps
    def forward(self, inputs, training, masks=None, ctx=None):
        x = inputs[0]
        dims = list(self.dimension) if self.dimension else list(range(1, x.dim()))
        return x / x.norm(2, dim=dims, keepdim=True).clamp_min(self.eps)


class L2Vertex(GraphVertex):
    JAVA = "L2Vertex"; FIELDS = ("eps",)
    def __init__(self, eps=1e-8): self.eps = eps
    def forward(self, inputs, training, masks=None, ctx=None):
        d = (inputs[0] - inputs[1]).reshape(inputs[0].shape[0], -1)
        return torch.sqrt((d * d).sum(1, keepdim=True) + self.eps)
    def output_type(self, *its): return InputType.feedForward(1)


class ReshapeVertex(GraphVertex):
    JAVA = "ReshapeVertex"; FIELDS = ("reshapeOrder", "newShape", "maskShape")
    def __init__(self, *newShape, reshapeOrder="c", maskShape=None):
        if len(newShape) == 1 and isinstance(newShape[0], (list, tuple)):
            newShape = newShape[0]
        self.newShape, self.reshapeOrder, self.maskShape = [int(s) for s in newShape], reshapeOrder, maskShape
    def forward(self, inputs, training, masks=None, ctx=None): return inputs[0].reshape(self.newShape)
    def output_type(self, *its):
        s = self.newShape
        if len(s) == 2: return InputType.feedForward(s[1])
        if len(s) == 3: return InputType.recurrent(s[1], s[2])
        if len(s) == 4: return InputType.convolutional(s[2], s[3], s[1])
        return its[0]


class PreprocessorVertex(GraphVertex):
    JAVA = "PreprocessorVertex"
    def __init__(self, preProcessor): self.preProcessor = preProcessor
    def forward(self, inputs, training, masks=None, ctx=None): return self.preProcessor.preProcess(inputs[0], inputs[0].shape[0], ctx)
    def output_type(self, *its): return self.preProcessor.output_type(its[0])
    def to_json(self): return {"@class": _G + self.JAVA, "preProcessor": self.preProcessor.to_json()}


class PoolHelperVertex(GraphVertex):
    """Strips the first row and column of a CNN activation (Keras/Caffe max-pool compatibility)."""
    JAVA = "PoolHelperVertex"
    def forward(self, inputs, training, masks=None, ctx=None): return inputs[0][:, :, 1:, 1:]
    def output_type(self, *its):
        a = its[0]
        return InputType.convolutional(a.height - 1, a.width - 1, a.channels, a.format)


class FrozenVertex(GraphVertex):
    JAVA = "FrozenVertex"
    def __init__(self, underlying): self.underlying = underlying
    @property
    def HAS_PARAMS(self): return self.underlying.HAS_PARAMS
    def param_specs(self): return self.underlying.param_specs()
    def output_type(self, *its): return self.underlying.output_type(*its)
    def forward(self, inputs, training, masks=None, ctx=None): return self.underlying.forward(inputs, False, masks, ctx)
    def to_json(self): return {"@class": _G + self.JAVA, "underlying": self.underlying.to_json()}


class DotProductAttentionVertex(GraphVertex):
    """Parameter-free attention over [queries, keys, values] inputs, each [mb, n, T]."""
    JAVA = "DotProductAttentionVertex"; FIELDS = ("scaleFactor", "dropoutProbability", "useCausalMask")
    def __init__(self, scaleFactor=None, dropoutProbability=0.0, useCausalMask=False):
        self.scaleFactor, self.dropoutProbability, self.useCausalMask = scaleFactor, dropoutProbability, useCausalMask
    def forward(self, inputs, training, masks=None, ctx=None):
        from ...ops import nnops
        q, k, v = (inputs + inputs[-1:] * 3)[:3]
        qq, kk, vv = (t.permute(0, 2, 1).unsqueeze(1) for t in (q, k, v))
        m = masks[1] if masks and len(masks) > 1 else None
        if self.useCausalMask:                       # query step t sees key steps <= t; folded with the key mask into one additive mask
            import torch
            add = torch.full((qq.shape[2], kk.shape[2]), float("-inf"), device=qq.device, dtype=torch.float32).triu(1)[None, None]
            if m is not None:
                add = add.masked_fill(m[:, None, None, :] == 0, float("-inf"))
            m = add
        o = nnops.attention(qq, kk, vv, m, self.scaleFactor, self.dropoutProbability, training)
        return o.squeeze(1).permute(0, 2, 1)
    def output_type(self, *its):
        return InputType.recurrent(its[-1].size, its[0].timeSeriesLength, its[0].format)


class AttentionVertex(GraphVertex):
    """Multi-head attention vertex with its own projection weights (``AttentionVertex.java``)."""
    JAVA = "AttentionVertex"; FIELDS = ("nInKeys", "nInValues", "nInQueries", "nOut", "headSize", "nHeads", "projectInput")
    def __init__(self, nInKeys=0, nInValues=0, nInQueries=0, nOut=0, headSize=0, nHeads=1, projectInput=True, weightInit=None):
        self.nInKeys, self.nInValues, self.nInQueries, self.nOut = nInKeys, nInValues, nInQueries, nOut
        self.nHeads, self.projectInput = nHeads, projectInput
        self.headSize = headSize or (nOut // max(nHeads, 1))
        self.weightInit = weightInit
    @property
    def HAS_PARAMS(self): return self.projectInput
    def param_specs(self):
        from .base import ParamSpec
        if not self.projectInput:
            return []
        h, d = self.nHeads, self.headSize
        return [ParamSpec("Wq", (h, d, self.nInQueries), "c", "weight", self.nInQueries, d),
                ParamSpec("Wk", (h, d, self.nInKeys), "c", "weight", self.nInKeys, d),
                ParamSpec("Wv", (h, d, self.nInValues), "c", "weight", self.nInValues, d),
                ParamSpec("Wo", (h * d, self.nOut), "c", "weight", h * d, self.nOut)]
    def forward(self, inputs, training, masks=None, ctx=None, p=None):
        from ..layers.attention import _mha
        q, k, v = (inputs + inputs[-1:] * 3)[:3]
        from ...ops import registry
        if not self.projectInput:
            return _mha(q, k, {}, 1, 0, False, masks[1] if masks and len(masks) > 1 else None, training)
        y = registry.get("multi_head_dot_product_attention").fn(q, k, v, p["Wq"], p["Wk"], p["Wv"], p["Wo"],
                                                                  masks[1] if masks and len(masks) > 1 else None, True)
        return y[0]
    def output_type(self, *its):
        return InputType.recurrent(self.nOut if self.projectInput else its[-1].size, its[0].timeSeriesLength, its[0].format)


_R = _G + "rnn."


class LastTimeStepVertex(GraphVertex):
    JAVA = "rnn.LastTimeStepVertex"; FIELDS = ("maskArrayInputName",)
    def __init__(self, maskArrayInputName=None): self.maskArrayInputName = maskArrayInputName
    def forward(self, inputs, training, masks=None, ctx=None):
        x = inputs[0]
        m = (ctx or {}).get("input_masks", {}).get(self.maskArrayInputName) if self.maskArrayInputName else None
        if m is None:
            return x[:, :, -1]
        idx = (m.long() * torch.arange(x.shape[2], device=x.device)).argmax(1)
        return x.gather(2, idx.reshape(-1, 1, 1).expand(-1, x.shape[1], 1)).squeeze(2)
    def output_type(self, *its): return InputType.feedForward(its[0].size)
    def mask_out(self, masks): return None


class DuplicateToTimeSeriesVertex(GraphVertex):
    JAVA = "rnn.DuplicateToTimeSeriesVertex"; FIELDS = ("inputName",)
    def __init__(self, inputName=None): self.inputName = inputName
    def forward(self, inputs, training, masks=None, ctx=None):
        T = (ctx or {}).get("input_T", {}).get(self.inputName) or (ctx or {}).get("rnn_T", 1)
        return inputs[0].unsqueeze(2).expand(-1, -1, int(T))
    def output_type(self, *its): return InputType.recurrent(its[0].size, -1)


class ReverseTimeSeriesVertex(GraphVertex):
    JAVA = "rnn.ReverseTimeSeriesVertex"; FIELDS = ("maskArrayInputName",)
    def __init__(self, maskArrayInputName=None): self.maskArrayInputName = maskArrayInputName
    def forward(self, inputs, training, masks=None, ctx=None):
        x = inputs[0]
        m = (ctx or {}).get("input_masks", {}).get(self.maskArrayInputName) if self.maskArrayInputName else None
        if m is None:
            return x.flip(2)
        T = x.shape[2]
        lens = m.long().sum(1)
        ar = torch.arange(T, device=x.device).unsqueeze(0)
        idx = torch.where(ar < lens.unsqueeze(1), lens.unsqueeze(1) - 1 - ar, ar)
        return x.gather(2, idx.unsqueeze(1).expand(-1, x.shape[1], -1))


VERTICES = {c.JAVA: c for c in (LayerVertex, ElementWiseVertex, MergeVertex, SubsetVertex, StackVertex, UnstackVertex, ScaleVertex,
                                ShiftVertex, L2NormalizeVertex, L2Vertex, ReshapeVertex, PreprocessorVertex, PoolHelperVertex,
                                FrozenVertex, DotProductAttentionVertex, AttentionVertex, LastTimeStepVertex,
                                DuplicateToTimeSeriesVertex, ReverseTimeSeriesVertex)}


def vertex_from_json(d):
    from .registry import layer_from_json
    name = d["@class"].split(".graph.", 1)[-1]
    cls = VERTICES[name]
    if cls is LayerVertex:
        conf = NeuralNetConfiguration.from_json(d["layerConf"])
        return LayerVertex(conf.layer, preprocessor_from_json(d.get("preProcessor")), conf)
    if cls is PreprocessorVertex:
        return PreprocessorVertex(preprocessor_from_json(d["preProcessor"]))
    if cls is FrozenVertex:
        return FrozenVertex(vertex_from_json(d["underlying"]))
    if cls in (SubsetVertex, UnstackVertex):
        return cls(d["from"], d.get("to", d.get("stackSize")))
    if cls is ReshapeVertex:
        return ReshapeVertex(d["newShape"], reshapeOrder=d.get("reshapeOrder", "c"), maskShape=d.get("maskShape"))
    return cls(**{k: v for k, v in d.items() if k in cls.FIELDS})


class ComputationGraphConfiguration:
    def __init__(self):
        self.vertices: dict = {}
        self.vertexInputs: dict = {}
        self.networkInputs: list = []
        self.networkOutputs: list = []
        self.backpropType = BackpropType.Standard
        self.tbpttFwdLength = self.tbpttBackLength = 20
        self.trainingWorkspaceMode = self.inferenceWorkspaceMode = WorkspaceMode.ENABLED
        self.cacheMode = CacheMode.NONE
        self.dataType = DataType.FLOAT
        self.computeDataType = None
        self.validateOutputLayerConfig = True
        self.iterationCount = self.epochCount = 0
        self.inputTypes = None
        self.defaultConfiguration = None
        self.topologicalOrder = None

    def topological_order(self):
        if self.topologicalOrder is not None:
            return self.topologicalOrder
        indeg = {v: 0 for v in self.vertices}
        out_edges = {n: [] for n in list(self.vertices) + self.networkInputs}
        for v, ins in self.vertexInputs.items():
            for i in ins:
                out_edges[i].append(v)
                if i in self.vertices:
                    indeg[v] += 1
        # Kahn's algorithm with insertion-order tie breaking (stable across save/load)
        ready = [v for v in self.vertices if indeg[v] == 0]
        order = []
        while ready:
            v = ready.pop(0)
            order.append(v)
            for o in out_edges[v]:
                indeg[o] -= 1
                if indeg[o] == 0:
                    ready.append(o)
        if len(order) != len(self.vertices):
            raise ValueError("graph has a cycle or a vertex with a missing input")
        self.topologicalOrder = order
        return order

    def to_dict(self):
        d = {"backpropType": self.backpropType, "cacheMode": self.cacheMode, "dataType": self.dataType.name,
             "epochCount": self.epochCount, "inferenceWorkspaceMode": self.inferenceWorkspaceMode,
             "iterationCount": self.iterationCount, "networkInputs": list(self.networkInputs),
             "networkOutputs": list(self.networkOutputs), "tbpttBackLength": self.tbpttBackLength,
             "tbpttFwdLength": self.tbpttFwdLength, "topologicalOrder": None, "topologicalOrderStr": self.topological_order(),
             "trainingWorkspaceMode": self.trainingWorkspaceMode, "validateOutputLayerConfig": self.validateOutputLayerConfig,
             "vertexInputs": {k: list(v) for k, v in self.vertexInputs.items()},
             "vertices": {k: v.to_json() for k, v in self.vertices.items()}}
        if self.computeDataType is not None:
            d["computeDataType"] = self.computeDataType.name
        return d

    def toJson(self):
        return jackson.dumps(self.to_dict())

    @staticmethod
    def fromJson(s):
        d = jackson.loads(s) if isinstance(s, str) else s
        c = ComputationGraphConfiguration()
        order = d.get("topologicalOrderStr")
        names = order if order else list(d["vertices"])
        for n in names:
            c.vertices[n] = vertex_from_json(d["vertices"][n])
        for n in d["vertices"]:
            if n not in c.vertices:
                c.vertices[n] = vertex_from_json(d["vertices"][n])
        c.vertexInputs = {k: list(v) for k, v in d["vertexInputs"].items()}
        c.networkInputs, c.networkOutputs = list(d["networkInputs"]), list(d["networkOutputs"])
        c.backpropType = d.get("backpropType", "Standard")
        c.tbpttFwdLength, c.tbpttBackLength = d.get("tbpttFwdLength", 20), d.get("tbpttBackLength", 20)
        c.dataType = DataType.from_name(d.get("dataType", "FLOAT"))
        if d.get("computeDataType"):
            c.computeDataType = DataType.from_name(d["computeDataType"])
        c.iterationCount, c.epochCount = d.get("iterationCount", 0), d.get("epochCount", 0)
        c.topologicalOrder = order
        return c

    def clone(self):
        return ComputationGraphConfiguration.fromJson(self.toJson())

    def __eq__(self, o):
        return isinstance(o, ComputationGraphConfiguration) and self.toJson() == o.toJson()


class GraphBuilder:
    def __init__(self, parent):
        self.parent = parent
        self.c = ComputationGraphConfiguration()
        self._inputTypes = None
        self._pp = {}

    def addInputs(self, *names):
        self.c.networkInputs.extend(names[0] if len(names) == 1 and isinstance(names[0], (list, tuple)) else names)
        return self

    def setInputTypes(self, *its):
        self._inputTypes = list(its)
        return self

    def addLayer(self, name, layer, *rest):
        pp = None
        if rest and not isinstance(rest[0], str) and rest[0] is not None and not isinstance(rest[0], (list, tuple)):
            pp, rest = rest[0], rest[1:]
        elif rest and rest[0] is None:
            rest = rest[1:]
        inputs = list(rest[0]) if len(rest) == 1 and isinstance(rest[0], (list, tuple)) else list(rest)
        layer = _unbuild(layer)
        layer.layerName = layer.layerName or name
        layer.apply_global(self.parent.g)
        if hasattr(layer, "resolved"):
            layer.resolved()
        if len(inputs) > 1:     # implicit merge, as the reference does
            mname = name + "-merge"
            self.c.vertices[mname] = MergeVertex()
            self.c.vertexInputs[mname] = inputs
            inputs = [mname]
        self.c.vertices[name] = LayerVertex(layer, pp, self.parent._conf_for(layer))
        self.c.vertexInputs[name] = inputs
        return self

    layer = addLayer

    def addVertex(self, name, vertex, *inputs):
        inputs = list(inputs[0]) if len(inputs) == 1 and isinstance(inputs[0], (list, tuple)) else list(inputs)
        self.c.vertices[name] = vertex
        self.c.vertexInputs[name] = inputs
        return self

    def removeVertex(self, name, removeConnections=True):
        self.c.vertices.pop(name, None)
        self.c.vertexInputs.pop(name, None)
        if removeConnections:
            for k, v in self.c.vertexInputs.items():
                self.c.vertexInputs[k] = [i for i in v if i != name]
        return self

    def inputPreProcessor(self, name, pp):
        self._pp[name] = pp
        return self

    def setOutputs(self, *names):
        self.c.networkOutputs = list(names[0]) if len(names) == 1 and isinstance(names[0], (list, tuple)) else list(names)
        return self

    def backpropType(self, t): self.c.backpropType = t; return self
    def tBPTTForwardLength(self, n): self.c.tbpttFwdLength = int(n); return self
    def tBPTTBackwardLength(self, n): self.c.tbpttBackLength = int(n); return self
    def tBPTTLength(self, n): self.c.tbpttFwdLength = self.c.tbpttBackLength = int(n); return self
    def validateOutputLayerConfig(self, b): self.c.validateOutputLayerConfig = b; return self
    def allowDisconnected(self, b): return self
    def allowNoOutput(self, b): return self

    def _infer_types(self, order):
        """Propagates InputTypes through the (possibly partial) graph, setting nIn and pre-processors on the way."""
        c = self.c
        types = dict(zip(c.networkInputs, self._inputTypes))
        for n in order:
            v = c.vertices[n]
            its = [types[i] for i in c.vertexInputs[n]]
            if isinstance(v, LayerVertex):
                it = its[0]
                pp = v.preProcessor if v.preProcessor is not None else self._pp.get(n)
                if pp is None:
                    pp = v.preProcessor = v.layer.preprocessor_for(it)
                if pp is not None:
                    it = pp.output_type(it)
                v.layer.setNIn(it, True)
                types[n] = v.layer.output_type(it)
            else:
                if isinstance(v, AttentionVertex) and not v.nInQueries:
                    v.nInQueries, v.nInKeys, v.nInValues = its[0].size, its[min(1, len(its) - 1)].size, its[-1].size
                types[n] = v.output_type(*its)
        return types

    def getLayerActivationTypes(self):
        """Output InputType of every vertex added so far (``GraphBuilder.getLayerActivationTypes``); needs setInputTypes."""
        if self._inputTypes is None:
            raise ValueError("setInputTypes(...) must be called before activation types can be computed")
        self.c.topologicalOrder = None
        types = self._infer_types(self.c.topological_order())
        self.c.topologicalOrder = None               # the graph is still being built
        return types

    def getVertices(self): return self.c.vertices

    def build(self):
        c, p = self.c, self.parent
        c.dataType, c.computeDataType = p._dataType, p._computeDataType
        c.trainingWorkspaceMode, c.inferenceWorkspaceMode, c.cacheMode = p._trainingWorkspaceMode, p._inferenceWorkspaceMode, p._cacheMode
        for n, pp in self._pp.items():
            c.vertices[n].preProcessor = pp
        for n, ins in c.vertexInputs.items():
            for i in ins:
                if i not in c.vertices and i not in c.networkInputs:
                    raise ValueError(f"vertex '{n}' has unknown input '{i}'")
        order = c.topological_order()
        if self._inputTypes is not None:
            self._infer_types(order)
            c.inputTypes = self._inputTypes
        for n in order:
            v = c.vertices[n]
            if isinstance(v, LayerVertex):
                v.conf.variables = [s.name for s in v.layer.param_specs()]
        return c
