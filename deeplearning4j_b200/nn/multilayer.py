"""``MultiLayerNetwork`` — sequential stack of layers trained by SGD-family updaters.

Parity: ``deeplearning4j-nn/.../nn/multilayer/MultiLayerNetwork.java`` — ``init`` ``:604``,
``fit`` ``:1677-1785``, truncated BPTT ``:2105-2147``, ``computeGradientAndScore``
``:2752-2826``, ``output`` ``:2290-2376``, ``rnnTimeStep``, ``evaluate``, ``score``.

Forward is a chain of differentiable torch/CUDA ops over views of the flat parameter buffer;
backward is autograd writing straight into views of the flat gradient buffer (each leaf's
``.grad`` *is* its gradient view), then one fused updater launch steps the parameters.
"""
from __future__ import annotations

import torch

from ..nd.ndarray import INDArray, wrap
from .conf.base import BackpropType
from .conf.neuralnet import MultiLayerConfiguration
from .network import BaseNetwork, _as_tensor
from ..utils.crash import guard_fit
from ..utils import nvtx as _nvtx


class MultiLayerNetwork(BaseNetwork):
    def __init__(self, conf: MultiLayerConfiguration | str, params=None):
        super().__init__()
        if isinstance(conf, str):
            conf = MultiLayerConfiguration.fromJson(conf)
        self.conf = conf
        self.layers = conf.layers()
        self._initial_params = params
        self._initialized = False
        self._rnn_state = {}
        self._tbptt_state = {}
        self.mask_features = None
        self.mask_labels = None
        self._input = None
        self._labels = None

    # ------------------------------------------------------------------ init
    def _owners(self):
        return [(str(i), l) for i, l in enumerate(self.layers)]

    def init(self, params=None, cloneParametersArray=True):
        if self._initialized and params is None:
            return self
        params = params if params is not None else self._initial_params
        seed = self.conf.confs[0].seed if self.conf.confs else 0
        self._init_params(params, cloneParametersArray, seed)
        self.iterationCount = self.conf.iterationCount
        self.epochCount = self.conf.epochCount
        self._initialized = True
        return self

    def getLayerWiseConfigurations(self):
        return self.conf

    def getnLayers(self):
        return len(self.layers)

    def getLayer(self, i):
        if isinstance(i, str):
            for l in self.layers:
                if l.layerName == i:
                    return l
            raise KeyError(i)
        return self.layers[i]

    def getLayers(self):
        return list(self.layers)

    def getOutputLayer(self):
        return self.layers[-1]

    def summary(self):
        lines = ["=" * 78, f"{'LayerName (LayerType)':<34}{'nIn,nOut':<14}{'TotalParams':<14}ParamsShape", "=" * 78]
        tot = 0
        for i, l in enumerate(self.layers):
            specs = l.param_specs()
            n = sum(s.numel for s in specs)
            tot += n
            shp = ", ".join(f"{s.name}:{{{','.join(map(str, s.shape))}}}" for s in specs) or "-"
            nio = f"{getattr(l, 'nIn', '-')},{getattr(l, 'nOut', '-')}"
            lines.append(f"{(l.layerName or 'layer' + str(i)) + ' (' + type(l).__name__ + ')':<34}{nio:<14}{n:<14}{shp}")
        lines += ["-" * 78, f"{'Total Parameters:':>30}  {tot}", "=" * 78]
        return "\n".join(lines)

    # ------------------------------------------------------------------ forward
    def _prep_input(self, x):
        x = _as_tensor(x, self.device)
        cd = self._compute_dtype()
        if x.dtype.is_floating_point and x.dtype != cd:
            x = x.to(cd)
        return x

    def _forward(self, x, training, upto=None, fmask=None, ctx=None, collect=None):
        ctx = ctx if ctx is not None else {}
        ctx.setdefault("minibatch", x.shape[0])
        n = len(self.layers) if upto is None else upto + 1
        pps = self.conf.inputPreProcessors
        mask = fmask
        cd = self._compute_dtype()
        for i in range(n):
            l = self.layers[i]
            if i in pps:
                x = pps[i].preProcess(x, ctx["minibatch"], ctx)
                mask = pps[i].feed_forward_mask(mask, ctx["minibatch"])
            p = self.param_views.get(str(i), {})
            if _nvtx._on:
                with _nvtx.range(f"layer {i} {type(l).__name__}"):
                    x = l.forward(p, x, training, mask, ctx)
            else:
                x = l.forward(p, x, training, mask, ctx)
            mask = l.feed_forward_mask(mask)
            if collect is not None:
                collect.append(x)
        return x

    def output(self, x, train=False, featuresMask=None, labelsMask=None):
        if hasattr(x, "next") and hasattr(x, "hasNext"):
            outs = []
            x.reset()
            for ds in x:
                outs.append(self.output(ds.getFeatures(), train).t)
            return INDArray(torch.cat(outs, 0))
        with torch.no_grad():
            y = self._forward(self._prep_input(x), bool(train), fmask=_as_tensor(featuresMask, self.device))
        return INDArray(y.float() if y.dtype in (torch.bfloat16, torch.float16) else y)

    def feedForward(self, x=None, train=False):
        x = self._prep_input(x if x is not None else self._input)
        acts = []
        with torch.no_grad():
            self._forward(x, bool(train), collect=acts)
        return [INDArray(x)] + [INDArray(a) for a in acts]

    def feedForwardToLayer(self, layerNum, x, train=False):
        acts = []
        with torch.no_grad():
            self._forward(self._prep_input(x), bool(train), upto=layerNum, collect=acts)
        return [INDArray(self._prep_input(x))] + [INDArray(a) for a in acts]

    def activateSelectedLayers(self, frm, to, x):
        x = self._prep_input(x)
        with torch.no_grad():
            ctx = {"minibatch": x.shape[0]}
            for i in range(frm, to + 1):
                if i in self.conf.inputPreProcessors:
                    x = self.conf.inputPreProcessors[i].preProcess(x, x.shape[0], ctx)
                x = self.layers[i].forward(self.param_views.get(str(i), {}), x, False, None, ctx)
        return INDArray(x)

    def predict(self, x):
        if hasattr(x, "getFeatures"):
            x = x.getFeatures()
        return self.output(x).t.argmax(dim=1).cpu().tolist()

    def labelProbabilities(self, x):
        return self.output(x)

    # ------------------------------------------------------------------ loss
    def _loss(self, x, labels, fmask=None, lmask=None, training=True, ctx=None):
        ctx = ctx if ctx is not None else {}
        out_layer = self.layers[-1]
        if not getattr(out_layer, "IS_OUTPUT", False):
            raise ValueError("last layer is not an output layer: cannot compute a score")
        self._forward(x, training, fmask=fmask, ctx=ctx)
        preout = ctx["preout"]
        loss = out_layer.score_from_preout(preout, labels, lmask, True, minibatch=x.shape[0])
        if hasattr(out_layer, "extra_score"):
            loss = loss + out_layer.extra_score(ctx, labels)
        return loss

    def computeGradientAndScore(self, features=None, labels=None, fmask=None, lmask=None):
        x = self._prep_input(features if features is not None else self._input)
        y = _as_tensor(labels if labels is not None else self._labels, self.device)
        self.flat_grads.zero_()
        loss = self._loss(x, y, _as_tensor(fmask, self.device), _as_tensor(lmask, self.device), True)
        loss.backward()
        reg = self._regularization_score()
        self._score = loss.detach() + (reg if reg is not None else 0.0)
        self._last_batch = x.shape[0]
        return self.gradient(), float(self._score)

    def _score_dataset(self, ds, training=False):
        x = self._prep_input(ds.getFeatures())
        y = _as_tensor(ds.getLabels(), self.device)
        with torch.no_grad():
            loss = self._loss(x, y, _as_tensor(ds.getFeaturesMaskArray(), self.device),
                              _as_tensor(ds.getLabelsMaskArray(), self.device), training)
            reg = self._regularization_score()
        return float(loss + (reg if reg is not None else 0.0))

    def scoreExamples(self, ds, addRegularizationTerms=True):
        x = self._prep_input(ds.getFeatures())
        y = _as_tensor(ds.getLabels(), self.device)
        with torch.no_grad():
            ctx = {}
            self._forward(x, False, ctx=ctx)
            s = self.layers[-1].score_array(ctx["preout"], y, _as_tensor(ds.getLabelsMaskArray(), self.device))
            if addRegularizationTerms:
                reg = self._regularization_score()
                if reg is not None:
                    s = s + reg
        return INDArray(s.reshape(-1, 1))

    # ------------------------------------------------------------------ fit
    def setInput(self, x): self._input = x
    def setLabels(self, y): self._labels = y
    def getInput(self): return self._input
    def getLabels(self): return self._labels

    def setLayerMaskArrays(self, fm, lm):
        self.mask_features, self.mask_labels = fm, lm

    def clearLayerMaskArrays(self):
        self.mask_features = self.mask_labels = None

    @guard_fit
    def fit(self, *args, **kw):
        """``fit(DataSetIterator[, epochs])``, ``fit(DataSet)``, ``fit(features, labels[, fmask, lmask])``."""
        if not self._initialized:
            self.init()
        a0 = args[0] if args else None
        if a0 is None:
            self._fit_arrays(self._input, self._labels)
        elif hasattr(a0, "getFeatures") and not hasattr(a0, "hasNext"):
            self._fit_batch(a0)
        elif hasattr(a0, "__iter__") and not isinstance(a0, (torch.Tensor, INDArray)) and not hasattr(a0, "shape"):
            epochs = args[1] if len(args) > 1 else kw.get("epochs", 1)
            self._fit_iterator(a0, epochs)
        else:
            self._fit_arrays(*args)
        return self

    def _fit_batch(self, ds):
        self._fit_arrays(ds.getFeatures(), ds.getLabels(), ds.getFeaturesMaskArray(), ds.getLabelsMaskArray())

    def _fit_arrays(self, features, labels, fmask=None, lmask=None):
        x = self._prep_input(features)
        y = _as_tensor(labels, self.device)
        fm, lm = _as_tensor(fmask, self.device), _as_tensor(lmask, self.device)
        if self.conf.backpropType == BackpropType.TruncatedBPTT and x.dim() == 3:
            self._fit_tbptt(x, y, fm, lm)
        else:
            self._train_step(x, y, fm, lm)

    def _train_step(self, x, y, fm=None, lm=None, ctx=None):
        no_masks = fm is None and lm is None
        if ctx and set(ctx.keys()) <= {"rnn_state_in"} and no_masks:
            # truncated BPTT segment: carried recurrent state becomes extra step inputs / outputs (CUDA-graph friendly)
            st_in = ctx.get("rnn_state_in") or {}
            keys = sorted(st_in.keys(), key=str)
            sizes = [len(st_in[k]) for k in keys]
            aux = {}

            def loss_fn(ts):
                pos, st = 2, {}
                for k, n in zip(keys, sizes):
                    st[k] = tuple(ts[pos:pos + n])
                    pos += n
                c = {"rnn_state_in": st}
                loss = self._loss(ts[0], ts[1], None, None, True, c)
                aux["rnn_state_out"] = c.get("rnn_state_out", {})
                return loss
            self._score = self._loss_backward([x, y] + [t for k in keys for t in st_in[k]], loss_fn, aux=aux)
            ctx["rnn_state_out"] = aux.get("rnn_state_out", {})
        else:
            self._score = self._loss_backward([x, y], lambda ts: self._loss(ts[0], ts[1], fm, lm, True, ctx),
                                              eager_ok=no_masks and not ctx)
        self._last_batch = x.shape[0]
        if self.listeners:
            self._fire("onGradientCalculation")
        with torch.no_grad():
            self._apply_update()
            if not self.flat_params.is_cuda or not self._grads_zeroed_by_kernel():
                self.flat_grads.zero_()
        self._iteration_done()

    def _grads_zeroed_by_kernel(self):
        from ..ops import native
        return native.available() and getattr(self.updater, "_fused_zeroes_grads", False)

    def _fit_tbptt(self, x, y, fm, lm):
        fwd = self.conf.tbpttFwdLength
        T = x.shape[2]
        n_sub = (T + fwd - 1) // fwd
        state = {}
        for i in range(n_sub):
            s, e = i * fwd, min((i + 1) * fwd, T)
            xs = x[:, :, s:e]
            ys = y[:, :, s:e] if y.dim() == 3 else (y[:, s:e] if y.dim() == 2 and y.shape[1] == T else y)
            fms = fm[:, s:e] if fm is not None else None
            lms = lm[:, s:e] if lm is not None else None
            ctx = {"rnn_state_in": state}
            self._train_step(xs, ys, fms, lms, ctx)
            state = {k: tuple(t.detach() for t in v) for k, v in ctx.get("rnn_state_out", {}).items()}
        self._tbptt_state = state

    def pretrain(self, it, epochs=1):
        for i, l in enumerate(self.layers):
            if hasattr(l, "pretrain_score"):
                self.pretrainLayer(i, it, epochs)

    def pretrainLayer(self, idx, it, epochs=1):
        if not self._initialized:
            self.init()
        layer = self.layers[idx]
        if not hasattr(layer, "pretrain_score"):
            return
        for _ in range(epochs):
            if hasattr(it, "reset"):
                it.reset()
            for ds in it:
                x = self._prep_input(ds.getFeatures())
                with torch.no_grad():
                    if idx > 0:
                        x = self._forward(x, False, upto=idx - 1)
                    if idx in self.conf.inputPreProcessors:
                        x = self.conf.inputPreProcessors[idx].preProcess(x, x.shape[0], {})
                loss = layer.pretrain_score(self.param_views[str(idx)], x)
                loss.backward()
                self._score = loss.detach()
                with torch.no_grad():
                    self._apply_update()
                    self.flat_grads.zero_()
                self._iteration_done()

    # ------------------------------------------------------------------ rnn inference state
    def rnnTimeStep(self, x):
        x = self._prep_input(x)
        squeeze = x.dim() == 2
        if squeeze:
            x = x.unsqueeze(2)
        ctx = {"rnn_state_in": self._rnn_state}
        with torch.no_grad():
            y = self._forward(x, False, ctx=ctx)
        self._rnn_state = ctx.get("rnn_state_out", {})
        if squeeze and y.dim() == 3:
            y = y[:, :, -1]
        return INDArray(y)

    def rnnClearPreviousState(self):
        self._rnn_state = {}
        self._tbptt_state = {}

    def rnnGetPreviousState(self, layer):
        l = self.layers[layer]
        for k, v in self._rnn_state.items():
            if k == id(l):
                return v
        return None

    def rnnSetPreviousState(self, layer, state):
        self._rnn_state[id(self.layers[layer])] = state

    # ------------------------------------------------------------------ evaluation
    def evaluate(self, it, labelsList=None, topN=1):
        from ..eval.classification import Evaluation
        return self.doEvaluation(it, Evaluation(labels=labelsList, topN=topN))[0]

    def evaluateRegression(self, it):
        from ..eval.regression import RegressionEvaluation
        return self.doEvaluation(it, RegressionEvaluation())[0]

    def evaluateROC(self, it, thresholdSteps=0):
        from ..eval.roc import ROC
        return self.doEvaluation(it, ROC(thresholdSteps))[0]

    def evaluateROCMultiClass(self, it, thresholdSteps=0):
        from ..eval.roc import ROCMultiClass
        return self.doEvaluation(it, ROCMultiClass(thresholdSteps))[0]

    def doEvaluation(self, it, *evals):
        if hasattr(it, "reset"):
            it.reset()
        for ds in it:
            out = self.output(ds.getFeatures(), False, ds.getFeaturesMaskArray())
            for e in evals:
                e.eval(ds.getLabels(), out, ds.getLabelsMaskArray())
        return list(evals)

    # ------------------------------------------------------------------ misc
    def clone(self):
        m = MultiLayerNetwork(self.conf.clone())
        m.device = self.device
        m.init(self.flat_params.clone(), False)
        if self.updater is not None:
            m._ensure_updater().setStateViewArray(self.updater.state.clone())
        return m

    def save(self, path, saveUpdater=True):
        from .serializer import ModelSerializer
        ModelSerializer.writeModel(self, path, saveUpdater)

    @staticmethod
    def load(path, loadUpdater=True):
        from .serializer import ModelSerializer
        return ModelSerializer.restoreMultiLayerNetwork(path, loadUpdater)

    def toComputationGraph(self):
        from .graph import ComputationGraph
        from .conf.neuralnet import NeuralNetConfiguration
        gb = NeuralNetConfiguration.Builder().graphBuilder().addInputs("in")
        prev = "in"
        for i, l in enumerate(self.layers):
            name = l.layerName or f"layer{i}"
            pp = self.conf.inputPreProcessors.get(i)
            gb.addLayer(name, l.clone(), pp, prev) if pp is not None else gb.addLayer(name, l.clone(), prev)
            prev = name
        gb.setOutputs(prev)
        cg = ComputationGraph(gb.build())
        cg.device = self.device
        cg.init(self.flat_params.clone(), False)
        return cg
