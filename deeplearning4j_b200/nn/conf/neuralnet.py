"""``NeuralNetConfiguration`` (+Builder / ListBuilder) and ``MultiLayerConfiguration``.

JSON field names and nesting follow ``nn/conf/MultiLayerConfiguration.java:66-95`` and
``nn/conf/NeuralNetConfiguration.java:72-99`` so that ``configuration.json`` written here has
the same shape as one written by DL4J (``confs[i].layer`` typed by ``@class``).
"""
from __future__ import annotations

import copy

from ...nd.dtype import DataType
from ...serde import jackson
from ..updaters import IUpdater, L1Regularization, L2Regularization, Sgd, WeightDecay
from ..weights import WeightInit, Distribution
from ..activations import Activation
from .base import (BackpropType, CacheMode, ConvolutionMode, GradientNormalization, InputType, Layer,
                   OptimizationAlgorithm, WorkspaceMode, to_dropout)
from .preprocessors import preprocessor_from_json


class NeuralNetConfiguration:
    """Per-layer configuration record (one entry of ``MultiLayerConfiguration.confs``)."""

    def __init__(self, layer=None, seed=0, dataType=DataType.FLOAT, miniBatch=True, minimize=True,
                 optimizationAlgo=OptimizationAlgorithm.STOCHASTIC_GRADIENT_DESCENT, cacheMode=CacheMode.NONE,
                 maxNumLineSearchIterations=5, stepFunction=None):
        self.layer = layer
        self.seed = seed
        self.dataType = dataType
        self.miniBatch = miniBatch
        self.minimize = minimize
        self.optimizationAlgo = optimizationAlgo
        self.cacheMode = cacheMode
        self.maxNumLineSearchIterations = maxNumLineSearchIterations
        self.stepFunction = stepFunction
        self.variables = []
        self.iterationCount = 0
        self.epochCount = 0

    def to_json(self):
        return {"cacheMode": self.cacheMode, "dataType": self.dataType.name, "epochCount": self.epochCount,
                "iterationCount": self.iterationCount, "layer": self.layer.to_json() if self.layer else None,
                "maxNumLineSearchIterations": self.maxNumLineSearchIterations, "miniBatch": self.miniBatch,
                "minimize": self.minimize, "optimizationAlgo": self.optimizationAlgo, "seed": self.seed,
                "stepFunction": self.stepFunction, "variables": list(self.variables)}

    @staticmethod
    def from_json(d):
        from .registry import layer_from_json
        c = NeuralNetConfiguration(layer_from_json(d.get("layer")), d.get("seed", 0),
                                   DataType.from_name(d.get("dataType", "FLOAT")), d.get("miniBatch", True),
                                   d.get("minimize", True), d.get("optimizationAlgo", "STOCHASTIC_GRADIENT_DESCENT"),
                                   d.get("cacheMode", "NONE"), d.get("maxNumLineSearchIterations", 5), d.get("stepFunction"))
        c.variables = list(d.get("variables") or [])
        c.iterationCount = d.get("iterationCount", 0)
        c.epochCount = d.get("epochCount", 0)
        return c

    # ------------------------------------------------------------------ builder
    class Builder:
        def __init__(self):
            self.g = {"activation": None, "weightInit": None, "biasInit": None, "gainInit": None, "updater": None,
                      "biasUpdater": None, "regularization": [], "regularizationBias": [], "dropOut": None,
                      "weightNoise": None, "gradientNormalization": None, "gradientNormalizationThreshold": None,
                      "convolutionMode": ConvolutionMode.Truncate, "constraints": None}
            self._seed = 0
            self._dataType = DataType.FLOAT
            self._computeDataType = None
            self._miniBatch = True
            self._minimize = True
            self._optimizationAlgo = OptimizationAlgorithm.STOCHASTIC_GRADIENT_DESCENT
            self._trainingWorkspaceMode = WorkspaceMode.ENABLED
            self._inferenceWorkspaceMode = WorkspaceMode.ENABLED
            self._cacheMode = CacheMode.NONE
            self._maxNumLineSearchIterations = 5

        # global hyper-parameters ------------------------------------------------
        def seed(self, s): self._seed = int(s); return self
        def dataType(self, dt): self._dataType = dt; return self
        def computeDataType(self, dt):
            """Extension: run layer math in this dtype (bf16) while parameters, gradients and
            updater state stay in ``dataType`` (fp32 master weights)."""
            self._computeDataType = dt; return self
        def miniBatch(self, b): self._miniBatch = b; return self
        def minimize(self, b): self._minimize = b; return self
        def optimizationAlgo(self, a): self._optimizationAlgo = a; return self
        def maxNumLineSearchIterations(self, n): self._maxNumLineSearchIterations = n; return self
        def trainingWorkspaceMode(self, m): self._trainingWorkspaceMode = m; return self
        def inferenceWorkspaceMode(self, m): self._inferenceWorkspaceMode = m; return self
        def cacheMode(self, m): self._cacheMode = m; return self
        def activation(self, a): self.g["activation"] = Activation.get(a); return self
        def weightInit(self, w):
            self.g["weightInit"] = WeightInit.get(w); return self
        def dist(self, d): return self.weightInit(d)
        def biasInit(self, b): self.g["biasInit"] = float(b); return self
        def gainInit(self, b): self.g["gainInit"] = float(b); return self
        def updater(self, u): self.g["updater"] = u; return self
        def biasUpdater(self, u): self.g["biasUpdater"] = u; return self
        def dropOut(self, d): self.g["dropOut"] = to_dropout(d); return self
        def weightNoise(self, w): self.g["weightNoise"] = w; return self
        def gradientNormalization(self, gn): self.g["gradientNormalization"] = gn; return self
        def gradientNormalizationThreshold(self, t): self.g["gradientNormalizationThreshold"] = float(t); return self
        def convolutionMode(self, m): self.g["convolutionMode"] = m; return self
        def constrainWeights(self, *c): self.g["constraints"] = list(c); return self
        constrainAllParameters = constrainWeights
        def _reg(self, key, r):
            self.g[key] = [x for x in self.g[key] if type(x) is not type(r)] + [r]; return self
        def l1(self, v): return self._reg("regularization", L1Regularization(v))
        def l2(self, v): return self._reg("regularization", L2Regularization(v))
        def l1Bias(self, v): return self._reg("regularizationBias", L1Regularization(v))
        def l2Bias(self, v): return self._reg("regularizationBias", L2Regularization(v))
        def weightDecay(self, v, applyLR=True): return self._reg("regularization", WeightDecay(v, applyLR))
        def weightDecayBias(self, v, applyLR=True): return self._reg("regularizationBias", WeightDecay(v, applyLR))
        def regularization(self, r): self.g["regularization"] = list(r); return self
        def regularizationBias(self, r): self.g["regularizationBias"] = list(r); return self

        # terminal builders ------------------------------------------------------
        def list(self, *layers):
            lb = ListBuilder(self)
            for l in layers:
                lb.layer(l)
            return lb

        def graphBuilder(self):
            from .graphconf import GraphBuilder
            return GraphBuilder(self)

        def layer(self, layer):
            self._single = layer
            return self

        def build(self):
            l = getattr(self, "_single", None)
            if l is not None:
                l = _unbuild(l)
                l.apply_global(self.g)
            return self._conf_for(l)

        def _conf_for(self, layer):
            return NeuralNetConfiguration(layer, self._seed, self._dataType, self._miniBatch, self._minimize,
                                          self._optimizationAlgo, self._cacheMode, self._maxNumLineSearchIterations)

        def globals_json(self):
            return self.g


def _unbuild(l):
    return l.build() if hasattr(l, "build") and not isinstance(l, Layer) else l


class ListBuilder:
    """``NeuralNetConfiguration.ListBuilder``."""

    def __init__(self, parent):
        self.parent = parent
        self.layers = {}
        self.preprocs = {}
        self._inputType = None
        self._backpropType = BackpropType.Standard
        self._tbpttFwd = 20
        self._tbpttBack = 20
        self._validateOutput = True
        self._overrideNIn = True

    def layer(self, *a):
        if len(a) == 2:
            idx, l = a
        else:
            idx, l = len(self.layers), a[0]
        self.layers[int(idx)] = _unbuild(l)
        return self

    def inputPreProcessor(self, idx, pp): self.preprocs[int(idx)] = pp; return self
    def setInputType(self, it): self._inputType = it; return self
    inputType = setInputType
    def backpropType(self, t): self._backpropType = t; return self
    def tBPTTForwardLength(self, n): self._tbpttFwd = int(n); return self
    def tBPTTBackwardLength(self, n): self._tbpttBack = int(n); return self
    def tBPTTLength(self, n): self._tbpttFwd = self._tbpttBack = int(n); return self
    def validateOutputLayerConfig(self, b): self._validateOutput = b; return self
    def overrideNinUponBuild(self, b): self._overrideNIn = b; return self

    def build(self):
        p = self.parent
        n = len(self.layers)
        if sorted(self.layers) != list(range(n)):
            raise ValueError("layer indices must be contiguous from 0")
        confs = []
        it = self._inputType
        for i in range(n):
            l = self.layers[i]
            l.apply_global(p.g)
            if hasattr(l, "resolved"):
                l.resolved()
            if it is not None:
                if i not in self.preprocs:
                    pp = l.preprocessor_for(it)
                    if pp is not None:
                        self.preprocs[i] = pp
                if i in self.preprocs:
                    it = self.preprocs[i].output_type(it)
                l.setNIn(it, self._overrideNIn)
                it = l.output_type(it)
            c = p._conf_for(l)
            c.variables = [s.name for s in l.param_specs()]
            confs.append(c)
        conf = MultiLayerConfiguration(confs, dict(self.preprocs), self._backpropType, self._tbpttFwd, self._tbpttBack,
                                       self._validateOutput, p._trainingWorkspaceMode, p._inferenceWorkspaceMode,
                                       p._cacheMode, p._dataType, self._inputType)
        conf.computeDataType = p._computeDataType
        if self._validateOutput:
            conf.validate_output()
        return conf


class MultiLayerConfiguration:
    def __init__(self, confs, inputPreProcessors=None, backpropType=BackpropType.Standard, tbpttFwdLength=20,
                 tbpttBackLength=20, validateOutputLayerConfig=True, trainingWorkspaceMode=WorkspaceMode.ENABLED,
                 inferenceWorkspaceMode=WorkspaceMode.ENABLED, cacheMode=CacheMode.NONE, dataType=DataType.FLOAT,
                 inputType=None):
        self.confs = confs
        self.inputPreProcessors = inputPreProcessors or {}
        self.backpropType = backpropType
        self.tbpttFwdLength, self.tbpttBackLength = tbpttFwdLength, tbpttBackLength
        self.validateOutputLayerConfig = validateOutputLayerConfig
        self.trainingWorkspaceMode, self.inferenceWorkspaceMode = trainingWorkspaceMode, inferenceWorkspaceMode
        self.cacheMode = cacheMode
        self.dataType = dataType
        self.inputType = inputType
        self.computeDataType = None
        self.iterationCount = 0
        self.epochCount = 0

    def getConf(self, i):
        return self.confs[i]

    def layers(self):
        return [c.layer for c in self.confs]

    def validate_output(self):
        from ..activations import ActivationSoftmax, ActivationSigmoid
        from ..losses import LossMCXENT, LossBinaryXENT
        last = self.confs[-1].layer if self.confs else None
        lf = getattr(last, "lossFunction", None)
        act = getattr(last, "activation", None)
        if isinstance(lf, LossMCXENT) and type(lf).__name__ in ("LossMCXENT", "LossNegativeLogLikelihood") \
                and act is not None and not isinstance(act, ActivationSoftmax) and getattr(last, "nOut", 2) > 1:
            raise ValueError("Invalid output layer configuration: MCXENT loss requires a softmax activation "
                             "(disable with validateOutputLayerConfig(false))")

    def to_dict(self):
        d = {"backpropType": self.backpropType, "cacheMode": self.cacheMode,
             "confs": [c.to_json() for c in self.confs], "dataType": self.dataType.name, "epochCount": self.epochCount,
             "inferenceWorkspaceMode": self.inferenceWorkspaceMode,
             "inputPreProcessors": {str(k): v.to_json() for k, v in sorted(self.inputPreProcessors.items())},
             "iterationCount": self.iterationCount, "tbpttBackLength": self.tbpttBackLength,
             "tbpttFwdLength": self.tbpttFwdLength, "trainingWorkspaceMode": self.trainingWorkspaceMode,
             "validateOutputLayerConfig": self.validateOutputLayerConfig}
        if self.computeDataType is not None:
            d["computeDataType"] = self.computeDataType.name
        return d

    def toJson(self):
        return jackson.dumps(self.to_dict())

    def toYaml(self):
        import yaml
        return yaml.safe_dump(self.to_dict(), sort_keys=True)

    @staticmethod
    def fromJson(s):
        d = jackson.loads(s) if isinstance(s, str) else s
        confs = [NeuralNetConfiguration.from_json(c) for c in d["confs"]]
        pps = {int(k): preprocessor_from_json(v) for k, v in (d.get("inputPreProcessors") or {}).items()}
        c = MultiLayerConfiguration(confs, pps, d.get("backpropType", "Standard"), d.get("tbpttFwdLength", 20),
                                    d.get("tbpttBackLength", 20), d.get("validateOutputLayerConfig", True),
                                    d.get("trainingWorkspaceMode", "ENABLED"), d.get("inferenceWorkspaceMode", "ENABLED"),
                                    d.get("cacheMode", "NONE"), DataType.from_name(d.get("dataType", "FLOAT")))
        c.iterationCount = d.get("iterationCount", 0)
        c.epochCount = d.get("epochCount", 0)
        if d.get("computeDataType"):
            c.computeDataType = DataType.from_name(d["computeDataType"])
        return c

    @staticmethod
    def fromYaml(s):
        import yaml
        return MultiLayerConfiguration.fromJson(yaml.safe_load(s))

    def clone(self):
        return MultiLayerConfiguration.fromJson(self.toJson())

    def __eq__(self, o):
        return isinstance(o, MultiLayerConfiguration) and self.toJson() == o.toJson()
