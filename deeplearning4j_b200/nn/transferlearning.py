"""Transfer learning (``deeplearning4j-nn/.../nn/transferlearning``): ``FineTuneConfiguration``,
``TransferLearning.Builder`` (MultiLayerNetwork), ``TransferLearning.GraphBuilder`` (ComputationGraph)
and ``TransferLearningHelper`` (featurise once through the frozen part, train only the rest).

A new network is always built (flat buffers are re-laid-out); parameters of every layer whose
parameter shapes are unchanged are copied over, the rest are freshly initialised.
"""
from __future__ import annotations

import copy

import torch

from ..data.dataset import DataSet
from .conf.graphconf import FrozenVertex, LayerVertex
from .conf.neuralnet import NeuralNetConfiguration
from .layers.core import FrozenLayer


class FineTuneConfiguration:
    """Overrides applied to every non-frozen layer (and used as defaults for added layers)."""
    _FIELDS = ("activation", "weightInit", "biasInit", "l1", "l2", "l1Bias", "l2Bias", "weightDecay", "dropOut", "updater",
               "biasUpdater", "gradientNormalization", "gradientNormalizationThreshold", "weightNoise", "constraints")

    def __init__(self, **kw):
        self.values = {k: v for k, v in kw.items() if v is not None}

    class Builder:
        def __init__(self): self.kw = {}
        def __getattr__(self, k):
            if k.startswith("_") or k in ("kw", "build"):
                raise AttributeError(k)
            def setter(*v):
                self.kw[k] = v[0] if len(v) == 1 else list(v)
                return self
            return setter
        def build(self): return FineTuneConfiguration(**self.kw)

    @staticmethod
    def builder(): return FineTuneConfiguration.Builder()

    def apply_to_layer(self, layer):
        target = layer.layer if isinstance(layer, FrozenLayer) else layer
        for k, v in self.values.items():
            if k in ("seed", "miniBatch", "backpropType", "tbpttFwdLength", "tbpttBackLength", "trainingWorkspaceMode", "inferenceWorkspaceMode"):
                continue
            if k == "activation" and not hasattr(target, "activation"):
                continue
            if hasattr(target, k) or k in self._FIELDS:
                try:
                    setattr(target, k, copy.deepcopy(v))
                except AttributeError:
                    pass
        if hasattr(target, "resolved"):
            target.resolved()

    def apply_to_builder(self, b):
        for k, v in self.values.items():
            fn = getattr(b, k, None)
            if callable(fn):
                fn(v)
        return b


def _copy_params(src_net, dst_net, pairs):
    """pairs: (src key prefix, dst key prefix).  Copies every parameter whose shape matches."""
    src, dst = src_net.paramTable(), dst_net.paramTable()
    with torch.no_grad():
        for sp, dp in pairs:
            for k, v in src.items():
                if not k.startswith(sp + "_"):
                    continue
                dk = dp + k[len(sp):]
                if dk in dst:
                    a, b = getattr(v, "t", v), getattr(dst[dk], "t", dst[dk])
                    if a.shape == b.shape:
                        b.copy_(a)
    if getattr(dst_net, "flat_shadow", None) is not None:
        dst_net._refresh_shadow()


class TransferLearning:
    class Builder:
        def __init__(self, origModel):
            self.orig = origModel
            conf = origModel.conf
            self.layers = [copy.deepcopy(c.layer) for c in conf.confs]
            self.source = list(range(len(self.layers)))          # index in the original net, None for new / re-initialised layers
            self.preprocs = dict(conf.inputPreProcessors)
            self.ftc = None
            self.frozenTill = -1
            self.inputType = conf.inputType
            self._validate = conf.validateOutputLayerConfig

        def fineTuneConfiguration(self, ftc): self.ftc = ftc; return self
        def setFeatureExtractor(self, layerNum): self.frozenTill = int(layerNum); return self
        def setInputPreProcessor(self, idx, pp): self.preprocs[int(idx)] = pp; return self
        def validateOutputLayerConfig(self, b): self._validate = b; return self

        def nOutReplace(self, layerNum, nOut, weightInit=None, weightInitNext=None):
            l = self.layers[layerNum]
            l.nOut = int(nOut)
            if weightInit is not None:
                l.weightInit = weightInit
                if hasattr(l, "resolved"):
                    l.resolved()
            self.source[layerNum] = None
            if layerNum + 1 < len(self.layers):
                nxt = self.layers[layerNum + 1]
                if hasattr(nxt, "nIn") and layerNum + 1 not in self.preprocs:
                    nxt.nIn = int(nOut)
                    self.source[layerNum + 1] = None
                    if weightInitNext is not None:
                        nxt.weightInit = weightInitNext
                        if hasattr(nxt, "resolved"):
                            nxt.resolved()
            return self

        def nInReplace(self, layerNum, nIn, weightInit=None):
            l = self.layers[layerNum]
            l.nIn = int(nIn)
            if weightInit is not None:
                l.weightInit = weightInit
            self.source[layerNum] = None
            return self

        def removeOutputLayer(self): return self.removeLayersFromOutput(1)

        def removeLayersFromOutput(self, n):
            for _ in range(n):
                self.preprocs.pop(len(self.layers) - 1, None)
                self.layers.pop()
                self.source.pop()
            return self

        def addLayer(self, layer):
            from .conf.neuralnet import _unbuild
            self.layers.append(_unbuild(layer))
            self.source.append(None)
            return self

        def build(self):
            from .multilayer import MultiLayerNetwork
            oc = self.orig.conf
            b = NeuralNetConfiguration.Builder()
            if oc.confs:
                b.seed(oc.confs[0].seed)
            if self.ftc is not None:
                self.ftc.apply_to_builder(b)
            if oc.computeDataType is not None:
                b.computeDataType(oc.computeDataType)
            lb = b.list()
            for i, l in enumerate(self.layers):
                if i <= self.frozenTill:
                    l = l if isinstance(l, FrozenLayer) else FrozenLayer(l)
                elif self.ftc is not None and self.source[i] is not None:
                    self.ftc.apply_to_layer(l)
                lb.layer(i, l)
            for i, pp in self.preprocs.items():
                if i < len(self.layers):
                    lb.inputPreProcessor(i, pp)
            if self.inputType is not None:
                lb.setInputType(self.inputType)
            lb.backpropType(oc.backpropType).tBPTTForwardLength(oc.tbpttFwdLength).tBPTTBackwardLength(oc.tbpttBackLength)
            lb.validateOutputLayerConfig(self._validate)
            net = MultiLayerNetwork(lb.build())
            net.device = self.orig.device
            net.init()
            _copy_params(self.orig, net, [(str(s), str(i)) for i, s in enumerate(self.source) if s is not None])
            return net

    class GraphBuilder:
        def __init__(self, origGraph):
            self.orig = origGraph
            self.c = origGraph.conf.clone()
            self.ftc = None
            self.frozen = set()
            self.reinit = set()
            self.new = set()

        def fineTuneConfiguration(self, ftc): self.ftc = ftc; return self

        def setFeatureExtractor(self, *names):
            """Freeze the named vertices and everything they depend on."""
            names = list(names[0]) if len(names) == 1 and isinstance(names[0], (list, tuple)) else list(names)
            stack = list(names)
            while stack:
                n = stack.pop()
                if n in self.frozen or n not in self.c.vertices:
                    continue
                self.frozen.add(n)
                stack.extend(self.c.vertexInputs.get(n, []))
            return self

        def nOutReplace(self, name, nOut, weightInit=None, weightInitNext=None):
            v = self.c.vertices[name]
            v.layer.nOut = int(nOut)
            if weightInit is not None:
                v.layer.weightInit = weightInit
                if hasattr(v.layer, "resolved"):
                    v.layer.resolved()
            self.reinit.add(name)
            for n, ins in self.c.vertexInputs.items():
                if name in ins and isinstance(self.c.vertices[n], LayerVertex) and hasattr(self.c.vertices[n].layer, "nIn"):
                    nl = self.c.vertices[n].layer
                    if self.c.vertices[n].preProcessor is None:
                        nl.nIn = int(nOut)
                    if weightInitNext is not None:
                        nl.weightInit = weightInitNext
                    self.reinit.add(n)
            return self

        def removeVertexKeepConnections(self, name):
            self.c.vertices.pop(name)
            self._kept_inputs = getattr(self, "_kept_inputs", {})
            self._kept_inputs[name] = self.c.vertexInputs.pop(name)
            self.c.networkOutputs = [o for o in self.c.networkOutputs if o != name]
            return self

        def removeVertexAndConnections(self, name):
            self.c.vertices.pop(name)
            self.c.vertexInputs.pop(name)
            for k, v in list(self.c.vertexInputs.items()):
                self.c.vertexInputs[k] = [i for i in v if i != name]
            self.c.networkOutputs = [o for o in self.c.networkOutputs if o != name]
            return self

        def addLayer(self, name, layer, *inputs):
            from .conf.neuralnet import _unbuild
            pp = None
            if inputs and not isinstance(inputs[0], (str, list, tuple)):
                pp, inputs = inputs[0], inputs[1:]
            inputs = list(inputs[0]) if len(inputs) == 1 and isinstance(inputs[0], (list, tuple)) else list(inputs)
            layer = _unbuild(layer)
            layer.layerName = layer.layerName or name
            self.c.vertices[name] = LayerVertex(layer, pp, None)
            self.c.vertexInputs[name] = inputs or getattr(self, "_kept_inputs", {}).get(name, [])
            self.new.add(name)
            return self

        def addVertex(self, name, vertex, *inputs):
            self.c.vertices[name] = vertex
            self.c.vertexInputs[name] = list(inputs)
            self.new.add(name)
            return self

        def setOutputs(self, *names): self.c.networkOutputs = list(names); return self
        def setInputTypes(self, *its): self.c.inputTypes = list(its); return self

        def build(self):
            from .graph import ComputationGraph
            oc = self.orig.conf
            b = NeuralNetConfiguration.Builder()
            if self.ftc is not None:
                self.ftc.apply_to_builder(b)
            if oc.computeDataType is not None:
                b.computeDataType(oc.computeDataType)
            gb = b.graphBuilder()
            gb.addInputs(*self.c.networkInputs)
            if self.c.inputTypes:
                gb.setInputTypes(*self.c.inputTypes)
            for name, v in self.c.vertices.items():
                ins = self.c.vertexInputs[name]
                inner = v.underlying if isinstance(v, FrozenVertex) else v
                if isinstance(inner, LayerVertex):
                    layer = inner.layer
                    if name in self.frozen:
                        layer = layer if isinstance(layer, FrozenLayer) else FrozenLayer(layer)
                    elif self.ftc is not None and name not in self.new:
                        self.ftc.apply_to_layer(layer)
                    gb.addLayer(name, layer, inner.preProcessor, *ins)
                    if len(ins) > 1 and name + "-merge" in gb.c.vertices and name + "-merge" in self.c.vertices:
                        pass
                else:
                    gb.addVertex(name, v, *ins)
            gb.setOutputs(*self.c.networkOutputs)
            gb.backpropType(oc.backpropType).tBPTTForwardLength(oc.tbpttFwdLength).tBPTTBackwardLength(oc.tbpttBackLength)
            gb.validateOutputLayerConfig(oc.validateOutputLayerConfig)
            net = ComputationGraph(gb.build())
            net.device = self.orig.device
            net.init()
            keep = [n for n in self.c.vertices if n not in self.new and n not in self.reinit]
            _copy_params(self.orig, net, [(n, n) for n in keep])
            return net


class TransferLearningHelper:
    """Splits a network at the frozen boundary: ``featurize`` runs the frozen part once per dataset,
    ``fitFeaturized`` trains only the unfrozen tail on the stored activations."""

    def __init__(self, net, frozenTill=None):
        from .multilayer import MultiLayerNetwork
        if not isinstance(net, MultiLayerNetwork):
            raise TypeError("TransferLearningHelper here supports MultiLayerNetwork; freeze ComputationGraph vertices with GraphBuilder.setFeatureExtractor")
        if frozenTill is not None:
            net = TransferLearning.Builder(net).setFeatureExtractor(frozenTill).build()
        self.net = net
        layers = net.conf.layers()
        self.frozenTill = max([i for i, l in enumerate(layers) if isinstance(l, FrozenLayer)], default=-1)
        if self.frozenTill < 0:
            raise ValueError("no frozen layers: pass frozenTill or freeze layers first")
        tail_layers = [copy.deepcopy(l) for l in layers[self.frozenTill + 1:]]
        lb = NeuralNetConfiguration.Builder().list()
        for i, l in enumerate(tail_layers):
            lb.layer(i, l)
        for i, pp in net.conf.inputPreProcessors.items():
            if i > self.frozenTill:
                lb.inputPreProcessor(i - self.frozenTill - 1, pp)
        lb.validateOutputLayerConfig(False)
        self.tail = MultiLayerNetwork(lb.build())
        self.tail.device = net.device
        self.tail.init()
        self._pairs = [(str(i), str(i - self.frozenTill - 1)) for i in range(self.frozenTill + 1, len(layers))]
        _copy_params(net, self.tail, self._pairs)

    def unfrozenMLN(self): return self.tail

    def featurize(self, ds):
        with torch.no_grad():
            acts = self.net.feedForwardToLayer(self.frozenTill, ds.getFeatures(), False)
        a = acts[-1]
        return DataSet(a, ds.getLabels(), None, ds.getLabelsMaskArray())

    def fitFeaturized(self, data):
        self.tail.fit(data)
        _copy_params(self.tail, self.net, [(b, a) for a, b in self._pairs])

    def outputFromFeaturized(self, features):
        return self.tail.output(features)
