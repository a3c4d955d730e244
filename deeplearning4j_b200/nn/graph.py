"""``ComputationGraph`` — DAG of layers and vertices with multiple inputs/outputs.

Parity: ``deeplearning4j-nn/.../nn/graph/ComputationGraph.java`` — ``init`` / topological order
``:474,499-560`` (parameters are flattened in topological order), ``fit`` ``:972-1170``, ``output``,
``rnnTimeStep`` ``:3615-3671``, truncated BPTT.  Execution walks the cached topological order; every
layer vertex runs its layer over views of the flat parameter buffer, and autograd supplies the backward pass.
"""
from __future__ import annotations

import torch

from ..nd.ndarray import INDArray
from .conf.base import BackpropType
from .conf.graphconf import AttentionVertex, ComputationGraphConfiguration, FrozenVertex, LayerVertex
from .network import BaseNetwork, _as_tensor


from .conf.graphconf import ElementWiseVertex
from ..utils.crash import guard_fit


class _VertexOwner:
    """Lets a parameterised non-layer vertex (AttentionVertex) take part in the updater machinery."""
    gradientNormalization = None
    constraints = None

    def __init__(self, vertex, default_updater):
        self.vertex, self._u = vertex, default_updater

    def param_specs(self): return self.vertex.param_specs()
    def updater_for(self, spec): return self._u
    def regularizers(self, spec): return []
    weightInit = None


class ComputationGraph(BaseNetwork):
    def __init__(self, conf: ComputationGraphConfiguration | str, params=None):
        super().__init__()
        if isinstance(conf, str):
            conf = ComputationGraphConfiguration.fromJson(conf)
        self.conf = conf
        self.order = conf.topological_order()
        self._initial_params = params
        self._initialized = False
        self._rnn_state = {}

    # ------------------------------------------------------------------ init
    def _owners(self):
        owners = []
        default_upd = None
        for n in self.order:
            v = self.conf.vertices[n]
            if isinstance(v, LayerVertex) and getattr(v.layer, "updater", None) is not None and default_upd is None:
                default_upd = v.layer.updater
        for n in self.order:
            v = self.conf.vertices[n]
            if isinstance(v, LayerVertex):
                if v.layer.param_specs():
                    owners.append((n, v.layer))
            elif isinstance(v, FrozenVertex) and isinstance(v.underlying, LayerVertex):
                from .layers.core import FrozenLayer
                if v.underlying.layer.param_specs():
                    owners.append((n, FrozenLayer(v.underlying.layer)))
            elif v.param_specs():
                from .updaters import Sgd
                owners.append((n, _VertexOwner(v, default_upd or Sgd())))
        return owners

    def init(self, params=None, cloneParametersArray=True):
        if self._initialized and params is None:
            return self
        params = params if params is not None else self._initial_params
        seed = 0
        for n in self.order:
            v = self.conf.vertices[n]
            if isinstance(v, LayerVertex):
                seed = v.conf.seed
                break
        self._init_params(params, cloneParametersArray, seed)
        self.iterationCount, self.epochCount = self.conf.iterationCount, self.conf.epochCount
        self._initialized = True
        return self

    def getConfiguration(self): return self.conf
    def getNumInputArrays(self): return len(self.conf.networkInputs)
    def getNumOutputArrays(self): return len(self.conf.networkOutputs)
    def getVertices(self): return [self.conf.vertices[n] for n in self.order]
    def getVertex(self, name): return self.conf.vertices[name]
    def getLayer(self, name):
        v = self.conf.vertices[name] if isinstance(name, str) else self.conf.vertices[self.order[name]]
        return v.layer if isinstance(v, LayerVertex) else None
    def getLayers(self): return [v.layer for v in self.getVertices() if isinstance(v, LayerVertex)]
    def getOutputLayer(self, i=0): return self.getLayer(self.conf.networkOutputs[i])
    def topologicalSortOrder(self): return list(self.order)

    def summary(self):
        lines = ["=" * 96, f"{'VertexName (VertexType)':<40}{'nIn,nOut':<14}{'TotalParams':<13}{'ParamsShape':<18}Vertex Inputs", "=" * 96]
        tot = 0
        for n in self.order:
            v = self.conf.vertices[n]
            specs = v.param_specs()
            cnt = sum(s.numel for s in specs)
            tot += cnt
            l = v.layer if isinstance(v, LayerVertex) else None
            nio = f"{getattr(l, 'nIn', '-')},{getattr(l, 'nOut', '-')}" if l is not None else "-"
            shp = ", ".join(f"{s.name}:{{{','.join(map(str, s.shape))}}}" for s in specs) or "-"
            tname = type(l).__name__ if l is not None else type(v).__name__
            lines.append(f"{n + ' (' + tname + ')':<40}{nio:<14}{cnt:<13}{shp:<18}{self.conf.vertexInputs.get(n)}")
        lines += ["-" * 96, f"{'Total Parameters:':>30}  {tot}", "=" * 96]
        return "\n".join(lines)

    # ------------------------------------------------------------------ forward
    def _prep(self, x):
        x = _as_tensor(x, self.device)
        cd = self._compute_dtype()
        if x.dtype.is_floating_point and x.dtype != cd:
            x = x.to(cd)
        return x

    def _inputs(self, inputs):
        if isinstance(inputs, dict):
            return {k: self._prep(v) for k, v in inputs.items()}
        if not isinstance(inputs, (list, tuple)):
            inputs = [inputs]
        return {n: self._prep(x) for n, x in zip(self.conf.networkInputs, inputs)}

    def _fusion_plan(self):
        """Peephole plan for the executor: ``BatchNormalization -> ActivationLayer(ReLU)`` and
        ``BatchNormalization -> ElementWiseVertex(Add) -> ActivationLayer(ReLU)`` chains whose intermediate results have no
        other consumer run as one fused normalise(+add)+ReLU step.  vertex name -> action tuple."""
        plan = getattr(self, "_fuse_plan", None)
        if plan is not None:
            return plan
        from .activations import ActivationReLU
        from .layers.conv import BatchNormalization
        from .layers.core import ActivationLayer
        conf = self.conf
        consumers = {}
        for n in self.order:
            for i in conf.vertexInputs[n]:
                consumers.setdefault(i, []).append(n)
        outs = set(conf.networkOutputs)

        def plain_layer(n, cls):
            v = conf.vertices.get(n)
            return isinstance(v, LayerVertex) and type(v.layer) is cls and v.preProcessor is None and n not in outs \
                and getattr(v.layer, "dropOut", None) is None

        def is_relu(n):
            a = conf.vertices[n].layer.activation if plain_layer(n, ActivationLayer) else None
            return isinstance(a, ActivationReLU) and a.max is None and not a.threshold and not a.negativeSlope

        plan = {}
        for n in self.order:
            if not plain_layer(n, BatchNormalization) or n in plan:
                continue
            cs = consumers.get(n, [])
            if len(cs) != 1:
                continue
            c = cs[0]
            if is_relu(c):
                plan[n] = ("bn_relu",)
                plan[c] = ("alias", n)
                continue
            v = conf.vertices[c]
            if isinstance(v, ElementWiseVertex) and v.op == "Add" and len(conf.vertexInputs[c]) == 2 and c not in outs and c not in plan:
                cc = consumers.get(c, [])
                if len(cc) == 1 and is_relu(cc[0]):
                    other = [i for i in conf.vertexInputs[c] if i != n]
                    if len(other) == 1:
                        plan[n] = ("defer",)
                        plan[c] = ("bn_add_relu", n, other[0])
                        plan[cc[0]] = ("alias", c)
        # convolution bias -> following batch norm: batch statistics cancel the bias in training, so the convolution runs
        # without it and the batch norm accounts for it in its running mean / inference shift
        from .activations import ActivationIdentity
        from .layers.conv import ConvolutionLayer
        bias_of = {}
        for n in self.order:
            v = conf.vertices.get(n)
            if not (isinstance(v, LayerVertex) and type(v.layer) is ConvolutionLayer and v.layer.hasBias and n not in outs
                    and isinstance(v.layer.activation, ActivationIdentity) and getattr(v.layer, "weightNoise", None) is None
                    and getattr(v.layer, "dropOut", None) is None):
                continue
            cs = consumers.get(n, [])
            if len(cs) == 1 and plain_layer(cs[0], BatchNormalization):
                plan[n] = ("conv_nobias",)
                bias_of[cs[0]] = n
        self._fuse_bias = bias_of
        self._fuse_plan = plan
        return plan

    def _forward(self, inputs: dict, training, fmasks=None, ctx=None, stop_at_preout=False):
        ctx = ctx if ctx is not None else {}
        fuse = self._fusion_plan() if ctx.get("fuse") else {}
        bias_of = self._fuse_bias if fuse else {}

        def pre_bias(bn_name):
            c = bias_of.get(bn_name)
            return None if c is None else self.param_views[c]["b"]
        acts = dict(inputs)
        masks = dict(fmasks or {})
        first = next(iter(inputs.values()))
        ctx.setdefault("minibatch", first.shape[0])
        ctx["input_masks"] = {k: v for k, v in masks.items() if v is not None}
        ctx["input_T"] = {k: v.shape[2] for k, v in inputs.items() if v.dim() == 3}
        preouts = ctx.setdefault("preouts", {})
        conf = self.conf
        for n in self.order:
            v = conf.vertices[n]
            ins = [acts[i] for i in conf.vertexInputs[n]]
            in_masks = [masks.get(i) for i in conf.vertexInputs[n]]
            act = fuse.get(n)
            extra = {}
            if act is not None and act[0] == "conv_nobias":
                act, extra = None, {"skip_bias": True}
            elif act is None and n in bias_of:
                extra = {"pre_bias": pre_bias(n)}
            if act is not None:
                if act[0] == "bn_relu":
                    y = v.layer.forward(self.param_views.get(n, {}), ins[0], training, in_masks[0], None, fuse_relu=True,
                                        pre_bias=pre_bias(n))
                elif act[0] == "defer":
                    y = ins[0]                      # normalised later, at the add vertex that consumes it
                elif act[0] == "bn_add_relu":
                    bn = conf.vertices[act[1]]
                    y = bn.layer.forward(self.param_views.get(act[1], {}), acts[act[1]], training, masks.get(act[1]), None,
                                         fuse_relu=True, residual=acts[act[2]], pre_bias=pre_bias(act[1]))
                else:                               # alias: the ReLU already happened upstream
                    y = acts[act[1]]
                masks[n] = in_masks[0]
                acts[n] = y
                continue
            if isinstance(v, LayerVertex):
                x, m = ins[0], in_masks[0]
                if v.preProcessor is not None:
                    x = v.preProcessor.preProcess(x, ctx["minibatch"], ctx)
                    m = v.preProcessor.feed_forward_mask(m, ctx["minibatch"])
                lctx = {"minibatch": ctx["minibatch"], "rnn_state_in": ctx.get("rnn_state_in", {}),
                        "rnn_state_out": ctx.setdefault("rnn_state_out", {})}
                y = v.layer.forward(self.param_views.get(n, {}), x, training, m, lctx, **extra)
                if "preout" in lctx:
                    preouts[n] = lctx["preout"]
                    for k in ("center_in", "centers"):
                        if k in lctx:
                            ctx.setdefault("extra", {}).setdefault(n, {})[k] = lctx[k]
                masks[n] = v.layer.feed_forward_mask(m)
            elif isinstance(v, AttentionVertex):
                y = v.forward(ins, training, in_masks, ctx, p=self.param_views.get(n, {}))
                masks[n] = in_masks[0]
            elif isinstance(v, FrozenVertex) and isinstance(v.underlying, LayerVertex):
                p = {k: t.detach() for k, t in self.param_views.get(n, {}).items()}
                y = v.underlying.layer.forward(p, ins[0], False, in_masks[0], {"minibatch": ctx["minibatch"]})
                masks[n] = in_masks[0]
            else:
                y = v.forward(ins, training, in_masks, ctx)
                masks[n] = v.mask_out(in_masks)
            acts[n] = y
        return acts

    def output(self, *inputs, train=False, featureMasks=None):
        if len(inputs) == 1 and hasattr(inputs[0], "hasNext"):
            it = inputs[0]
            it.reset()
            outs = [self.output(*([ds.getFeatures()] if not isinstance(ds.getFeatures(), list) else ds.getFeatures())) for ds in it]
            return [INDArray(torch.cat([o[i].t for o in outs])) for i in range(len(outs[0]))]
        if len(inputs) == 2 and isinstance(inputs[0], bool):
            train, inputs = inputs[0], inputs[1:]
        ins = self._inputs(inputs[0] if len(inputs) == 1 and isinstance(inputs[0], (list, tuple, dict)) else list(inputs))
        fm = None
        if featureMasks is not None:
            fm = {n: _as_tensor(m, self.device) for n, m in zip(self.conf.networkInputs, featureMasks)}
        with torch.no_grad():
            acts = self._forward(ins, bool(train), fm)
        return [INDArray(acts[o].float() if acts[o].dtype in (torch.bfloat16, torch.float16) else acts[o]) for o in self.conf.networkOutputs]

    def outputSingle(self, *inputs, train=False):
        return self.output(*inputs, train=train)[0]

    def feedForward(self, inputs=None, train=False):
        ins = self._inputs(inputs)
        with torch.no_grad():
            acts = self._forward(ins, bool(train))
        return {k: INDArray(v) for k, v in acts.items()}

    # ------------------------------------------------------------------ loss
    def _loss(self, ins, labels, fmasks=None, lmasks=None, training=True, ctx=None):
        ctx = ctx if ctx is not None else {}
        ctx.setdefault("fuse", True)      # only the outputs are read here, so fused chains may skip intermediate activations
        self._forward(ins, training, fmasks, ctx)
        total = None
        mb = ctx["minibatch"]
        for i, name in enumerate(self.conf.networkOutputs):
            layer = self.getLayer(name)
            if layer is None or not getattr(layer, "IS_OUTPUT", False):
                continue
            lm = lmasks[i] if lmasks is not None and i < len(lmasks) else None
            l = layer.score_from_preout(ctx["preouts"][name], labels[i], lm, True, minibatch=mb)
            if hasattr(layer, "extra_score"):
                l = l + layer.extra_score(ctx["extra"][name], labels[i])
            total = l if total is None else total + l
        if total is None:
            raise ValueError("no output layer with a loss function among the network outputs")
        return total

    def _labels(self, labels):
        if not isinstance(labels, (list, tuple)):
            labels = [labels]
        return [_as_tensor(l, self.device) for l in labels]

    def computeGradientAndScore(self, inputs, labels, fmasks=None, lmasks=None):
        self.flat_grads.zero_()
        loss = self._loss(self._inputs(inputs), self._labels(labels))
        loss.backward()
        reg = self._regularization_score()
        self._score = loss.detach() + (reg if reg is not None else 0.0)
        return self.gradient(), float(self._score)

    def _score_dataset(self, ds, training=False):
        f, l = ds.getFeatures(), ds.getLabels()
        with torch.no_grad():
            loss = self._loss(self._inputs(f), self._labels(l), training=training)
            reg = self._regularization_score()
        return float(loss + (reg if reg is not None else 0.0))

    # ------------------------------------------------------------------ fit
    @guard_fit
    def fit(self, *args, **kw):
        if not self._initialized:
            self.init()
        a0 = args[0] if args else None
        if hasattr(a0, "getFeatures") and not hasattr(a0, "hasNext"):
            self._fit_batch(a0)
        elif hasattr(a0, "__iter__") and not isinstance(a0, (torch.Tensor, INDArray, list, tuple, dict)) and not hasattr(a0, "shape"):
            self._fit_iterator(a0, args[1] if len(args) > 1 else kw.get("epochs", 1))
        else:
            self._fit_arrays(args[0], args[1], *(args[2:]))
        return self

    def _fit_batch(self, ds):
        f, l = ds.getFeatures(), ds.getLabels()
        if hasattr(ds, "getFeaturesMaskArrays"):
            fm, lm = ds.getFeaturesMaskArrays(), ds.getLabelsMaskArrays()
        else:
            fm = [ds.getFeaturesMaskArray()] if ds.getFeaturesMaskArray() is not None else None
            lm = [ds.getLabelsMaskArray()] if ds.getLabelsMaskArray() is not None else None
        self._fit_arrays(f, l, fm, lm)

    def _fit_arrays(self, inputs, labels, fmasks=None, lmasks=None):
        ins = self._inputs(inputs)
        labs = self._labels(labels)
        fm = {n: _as_tensor(m, self.device) for n, m in zip(self.conf.networkInputs, fmasks)} if fmasks else None
        lm = [_as_tensor(m, self.device) for m in lmasks] if lmasks else None
        if self.conf.backpropType == BackpropType.TruncatedBPTT and any(x.dim() == 3 for x in ins.values()):
            self._fit_tbptt(ins, labs, fm, lm)
        else:
            self._train_step(ins, labs, fm, lm)

    def _train_step(self, ins, labs, fm=None, lm=None, ctx=None):
        names = list(ins.keys())
        n_in = len(names)

        n_lab = len(labs)
        no_masks = fm is None and (lm is None or all(m is None for m in lm))
        if ctx and set(ctx.keys()) <= {"rnn_state_in"} and no_masks:
            # truncated BPTT segment: the carried recurrent state travels as extra inputs / outputs of the step, so the
            # segment can replay from a CUDA graph like a stateless step
            st_in = ctx.get("rnn_state_in") or {}
            keys = sorted(st_in.keys(), key=str)
            sizes = [len(st_in[k]) for k in keys]
            aux = {}

            def loss_fn(ts):
                pos, st = n_in + n_lab, {}
                for k, n in zip(keys, sizes):
                    st[k] = tuple(ts[pos:pos + n])
                    pos += n
                c = {"rnn_state_in": st}
                loss = self._loss(dict(zip(names, ts[:n_in])), list(ts[n_in:n_in + n_lab]), None, None, True, c)
                aux["rnn_state_out"] = c.get("rnn_state_out", {})
                return loss
            tensors = [ins[n] for n in names] + list(labs) + [t for k in keys for t in st_in[k]]
            self._score = self._loss_backward(tensors, loss_fn, aux=aux)
            ctx["rnn_state_out"] = aux.get("rnn_state_out", {})
        else:
            def loss_fn(ts):
                return self._loss(dict(zip(names, ts[:n_in])), list(ts[n_in:]), fm, lm, True, ctx)
            self._score = self._loss_backward([ins[n] for n in names] + list(labs), loss_fn, eager_ok=no_masks and not ctx)
        self._last_batch = next(iter(ins.values())).shape[0]
        if self.listeners:
            self._fire("onGradientCalculation")
        with torch.no_grad():
            self._apply_update()
            from ..ops import native
            if not (self.flat_params.is_cuda and native.available() and getattr(self.updater, "_fused_zeroes_grads", False)):
                self.flat_grads.zero_()
        self._iteration_done()

    def _fit_tbptt(self, ins, labs, fm, lm):
        fwd = self.conf.tbpttFwdLength
        T = max(x.shape[2] for x in ins.values() if x.dim() == 3)
        state = {}
        for s in range(0, T, fwd):
            e = min(s + fwd, T)
            sub_in = {k: (v[:, :, s:e] if v.dim() == 3 else v) for k, v in ins.items()}
            sub_lab = [(l[:, :, s:e] if l.dim() == 3 else (l[:, s:e] if l.dim() == 2 and l.shape[1] == T else l)) for l in labs]
            sub_fm = {k: v[:, s:e] for k, v in fm.items()} if fm else None
            sub_lm = [m[:, s:e] if m is not None else None for m in lm] if lm else None
            ctx = {"rnn_state_in": state}
            self._train_step(sub_in, sub_lab, sub_fm, sub_lm, ctx)
            state = {k: tuple(t.detach() for t in v) for k, v in ctx.get("rnn_state_out", {}).items()}

    # ------------------------------------------------------------------ rnn state
    def rnnTimeStep(self, *inputs):
        ins = self._inputs(list(inputs))
        squeeze = all(v.dim() == 2 for v in ins.values())
        ins = {k: (v.unsqueeze(2) if v.dim() == 2 else v) for k, v in ins.items()}
        ctx = {"rnn_state_in": self._rnn_state}
        with torch.no_grad():
            acts = self._forward(ins, False, None, ctx)
        self._rnn_state = ctx.get("rnn_state_out", {})
        outs = [acts[o] for o in self.conf.networkOutputs]
        return [INDArray(o[:, :, -1] if squeeze and o.dim() == 3 else o) for o in outs]

    def rnnClearPreviousState(self):
        self._rnn_state = {}

    # ------------------------------------------------------------------ evaluation / misc
    def evaluate(self, it, labelsList=None, topN=1):
        from ..eval.classification import Evaluation
        return self.doEvaluation(it, Evaluation(labels=labelsList, topN=topN))[0]

    def evaluateRegression(self, it):
        from ..eval.regression import RegressionEvaluation
        return self.doEvaluation(it, RegressionEvaluation())[0]

    def evaluateROC(self, it, thresholdSteps=0):
        from ..eval.roc import ROC
        return self.doEvaluation(it, ROC(thresholdSteps))[0]

    def doEvaluation(self, it, *evals):
        if hasattr(it, "reset"):
            it.reset()
        for ds in it:
            f = ds.getFeatures()
            out = self.output(f if isinstance(f, list) else [f])[0]
            l = ds.getLabels()
            l = l[0] if isinstance(l, list) else l
            lm = ds.getLabelsMaskArray(0) if hasattr(ds, "getLabelsMaskArrays") and ds.getLabelsMaskArrays() else (
                ds.getLabelsMaskArray() if hasattr(ds, "getLabelsMaskArray") and not hasattr(ds, "getLabelsMaskArrays") else None)
            for e in evals:
                e.eval(l, out, lm)
        return list(evals)

    def clone(self):
        g = ComputationGraph(self.conf.clone())
        g.device = self.device
        g.init(self.flat_params.clone(), False)
        if self.updater is not None:
            g._ensure_updater().setStateViewArray(self.updater.state.clone())
        return g

    def save(self, path, saveUpdater=True):
        from .serializer import ModelSerializer
        ModelSerializer.writeModel(self, path, saveUpdater)

    @staticmethod
    def load(path, loadUpdater=True):
        from .serializer import ModelSerializer
        return ModelSerializer.restoreComputationGraph(path, loadUpdater)
