"""SameDiff training: ``TrainingConfig``, the flat-buffer training state, ``fit`` and ``History``.

Parity: ``autodiff/samediff/TrainingConfig.java:44-161``, ``SameDiff.fitHelper`` ``:1963-2212`` and
``internal/TrainingSession.java:73-271``.  The reference keeps one ``GradientUpdater`` per variable
and applies it as soon as that variable's gradient appears; here all trainable variables are views
of one flat fp32 buffer (plus a bf16 shadow used by the tensor-core kernels), gradients land in the
matching flat buffer through autograd, and one fused kernel applies regularisation, the updater and
the step for every variable.  Data-parallel hooks (``gradient_hook``) see the flat gradient
between backward and the update, which is where bucketed exchange overlaps.
"""
from __future__ import annotations

import time

import torch

from ..nd.dtype import DataType
from ..nn.conf.base import ParamSpec
from ..nn.updater import MultiLayerUpdater, ParamEntry
from ..nn.updaters import IUpdater, L1Regularization, L2Regularization, Regularization, Sgd, WeightDecay, updater_from_json, regularization_from_json
from ..serde import jackson
from .core import SDVariable, VariableType, _tensor


class TrainingConfig:
    def __init__(self, updater=None, regularization=None, minimize=True, dataSetFeatureMapping=None, dataSetLabelMapping=None,
                 dataSetFeatureMaskMapping=None, dataSetLabelMaskMapping=None, lossVariables=None, computeDataType=None,
                 iterationCount=0, epochCount=0, trainEvaluations=None, validationEvaluations=None, cudaGraphs=False):
        self.cudaGraphs = bool(cudaGraphs)      # replay forward + backward from a captured CUDA graph (runtime option, not serialised)
        self.updater = updater or Sgd()
        self.regularization = list(regularization or [])
        self.minimize = minimize
        self.dataSetFeatureMapping = list(dataSetFeatureMapping or [])
        self.dataSetLabelMapping = list(dataSetLabelMapping or [])
        self.dataSetFeatureMaskMapping = list(dataSetFeatureMaskMapping or [])
        self.dataSetLabelMaskMapping = list(dataSetLabelMaskMapping or [])
        self.lossVariables = list(lossVariables or [])
        self.computeDataType = computeDataType
        self.iterationCount, self.epochCount = iterationCount, epochCount
        self.trainEvaluations = trainEvaluations or {}
        self.validationEvaluations = validationEvaluations or {}

    @staticmethod
    def builder():
        return _TCBuilder()

    Builder = builder

    def placeholders_from(self, ds):
        ph = {}
        feats = ds.getFeatures()
        labs = ds.getLabels()
        feats = feats if isinstance(feats, list) else [feats]
        labs = labs if isinstance(labs, list) else [labs]
        for n, a in zip(self.dataSetFeatureMapping, feats):
            ph[n] = a
        for n, a in zip(self.dataSetLabelMapping, labs):
            if a is not None:
                ph[n] = a
        if self.dataSetFeatureMaskMapping:
            fm = ds.getFeaturesMaskArrays() if hasattr(ds, "getFeaturesMaskArrays") else [ds.getFeaturesMaskArray()]
            for n, a in zip(self.dataSetFeatureMaskMapping, fm or []):
                if a is not None:
                    ph[n] = a
        if self.dataSetLabelMaskMapping:
            lm = ds.getLabelsMaskArrays() if hasattr(ds, "getLabelsMaskArrays") else [ds.getLabelsMaskArray()]
            for n, a in zip(self.dataSetLabelMaskMapping, lm or []):
                if a is not None:
                    ph[n] = a
        return ph

    def toJson(self):
        d = {"@class": "org.nd4j.autodiff.samediff.TrainingConfig",
             "dataSetFeatureMapping": self.dataSetFeatureMapping, "dataSetFeatureMaskMapping": self.dataSetFeatureMaskMapping,
             "dataSetLabelMapping": self.dataSetLabelMapping, "dataSetLabelMaskMapping": self.dataSetLabelMaskMapping,
             "epochCount": self.epochCount, "iterationCount": self.iterationCount, "lossVariables": self.lossVariables,
             "minimize": self.minimize, "regularization": [r.to_json() for r in self.regularization],
             "updater": self.updater.to_json()}
        if self.computeDataType is not None:
            d["computeDataType"] = self.computeDataType.name
        return jackson.dumps(d)

    @staticmethod
    def fromJson(s):
        d = jackson.loads(s)
        tc = TrainingConfig(updater_from_json(d["updater"]), [regularization_from_json(r) for r in d.get("regularization") or []],
                            d.get("minimize", True), d.get("dataSetFeatureMapping"), d.get("dataSetLabelMapping"),
                            d.get("dataSetFeatureMaskMapping"), d.get("dataSetLabelMaskMapping"), d.get("lossVariables"),
                            DataType.from_name(d["computeDataType"]) if d.get("computeDataType") else None,
                            d.get("iterationCount", 0), d.get("epochCount", 0))
        return tc


class _TCBuilder:
    def __init__(self):
        self.kw = {"regularization": []}

    def updater(self, u): self.kw["updater"] = u; return self
    def l1(self, v): self.kw["regularization"].append(L1Regularization(v)); return self
    def l2(self, v): self.kw["regularization"].append(L2Regularization(v)); return self
    def weightDecay(self, v, applyLR=True): self.kw["regularization"].append(WeightDecay(v, applyLR)); return self
    def regularization(self, *r): self.kw["regularization"] = list(r[0]) if len(r) == 1 and isinstance(r[0], (list, tuple)) else list(r); return self
    def addRegularization(self, *r): self.kw["regularization"].extend(r); return self
    def minimize(self, *a):
        if a and isinstance(a[0], bool):
            self.kw["minimize"] = a[0]
        else:
            self.kw["lossVariables"] = list(a)
        return self
    def dataSetFeatureMapping(self, *n): self.kw["dataSetFeatureMapping"] = list(n[0]) if len(n) == 1 and isinstance(n[0], (list, tuple)) else list(n); return self
    def dataSetLabelMapping(self, *n): self.kw["dataSetLabelMapping"] = list(n[0]) if len(n) == 1 and isinstance(n[0], (list, tuple)) else list(n); return self
    def dataSetFeatureMaskMapping(self, *n): self.kw["dataSetFeatureMaskMapping"] = list(n[0]) if len(n) == 1 and isinstance(n[0], (list, tuple)) else list(n); return self
    def dataSetLabelMaskMapping(self, *n): self.kw["dataSetLabelMaskMapping"] = list(n[0]) if len(n) == 1 and isinstance(n[0], (list, tuple)) else list(n); return self
    def markLabelsUnused(self): self.kw["dataSetLabelMapping"] = []; return self
    def computeDataType(self, dt): self.kw["computeDataType"] = dt; return self
    def cudaGraphs(self, on=True): self.kw["cudaGraphs"] = bool(on); return self
    def trainEvaluation(self, var, labelIndex, *evals): self.kw.setdefault("trainEvaluations", {})[getattr(var, "name", var)] = (labelIndex, list(evals)); return self
    def validationEvaluation(self, var, labelIndex, *evals): self.kw.setdefault("validationEvaluations", {})[getattr(var, "name", var)] = (labelIndex, list(evals)); return self
    def skipBuilderValidation(self, b): return self
    def build(self): return TrainingConfig(**self.kw)


class _VarOwner:
    """Adapter that lets a SameDiff variable sit in the DL4J updater machinery as a one-parameter 'layer'."""
    gradientNormalization = None
    constraints = None

    def __init__(self, tc):
        self.tc = tc

    def updater_for(self, spec):
        return self.tc.updater

    def regularizers(self, spec):
        return self.tc.regularization if spec.kind == "weight" else []


class _ShadowParam(torch.autograd.Function):
    """Presents the low-precision shadow of a master parameter to the graph; the gradient flows back to
    the fp32 leaf (whose ``.grad`` is its view of the flat gradient buffer)."""

    @staticmethod
    def forward(ctx, leaf, shadow):
        # kernels that accumulate straight into the master gradient return no gradient for the shadow; without this
        # autograd would hand backward() a zero tensor, which costs a fill, a cast and an accumulate per parameter
        ctx.set_materialize_grads(False)
        ctx.leaf = leaf
        return shadow.view_as(shadow)

    @staticmethod
    def backward(ctx, g):
        # this node runs once every consumer of the parameter has run its backward: the parameter's gradient is final
        leaf = ctx.leaf
        cb = getattr(leaf, "_grad_ready", None)
        if cb is None:
            return (None if g is None else g.float()), None
        if g is not None:
            leaf.grad.add_(g)            # accumulate here (not in AccumulateGrad, which runs later) so that "final" holds
        cb(leaf)
        return None, None


class TrainingState:
    def __init__(self, sd, alloc=None):
        self.sd, self.tc = sd, sd.trainingConfig
        self.gradient_hook = None
        self.score = None
        self.updater = None
        self._build(alloc)

    def reallocate(self, alloc):
        """Move the flat buffers to memory obtained from ``alloc(numel, dtype, device)`` (e.g. symmetric
        memory for peer access), keeping parameter values and updater state."""
        old_state = self.updater.state.clone() if self.updater is not None else None
        self._build(alloc)
        if old_state is not None and old_state.numel() == self.updater.state.numel():
            self.updater.state.copy_(old_state)

    def _build(self, alloc=None):
        sd, tc = self.sd, self.tc
        dev = sd.device
        if alloc is None:
            alloc = lambda n, dt, d: torch.zeros(max(int(n), 1), dtype=dt, device=d)
        owner = _VarOwner(tc)
        entries, off = [], 0
        names = []
        for i, v in enumerate(sd.trainableVariables()):
            arr = sd.arrays[v.name]
            kind = "weight" if arr.dim() >= 2 else "bias"
            spec = ParamSpec(v.name, tuple(arr.shape), "c", kind)
            entries.append(ParamEntry(i, owner, spec, off, v.name))
            names.append(v.name)
            off += (spec.numel + 63) // 64 * 64      # every variable starts on a 256-byte boundary (vector / TMA access)
        self.entries, self.names = entries, names
        self.flat_params = alloc(off, torch.float32, dev)
        self.flat_grads = alloc(off, torch.float32, dev)
        self.flat_grads.zero_()
        self.views, self.compute_views = {}, {}
        cd = tc.computeDataType.to_torch() if tc.computeDataType is not None else torch.float32
        self.compute_dtype = cd
        mixed = cd != torch.float32 and dev.type == "cuda"
        self.flat_shadow, self.shadow_offsets = None, None
        if mixed:
            offs, so = [], 0
            for e in entries:
                offs.append(so)
                so += (e.spec.numel + 63) // 64 * 64
            self.shadow_offsets = offs
            self.flat_shadow = alloc(so, cd, dev)
        with torch.no_grad():
            self.flat_params.zero_()
            for i, e in enumerate(entries):
                seg = self.flat_params[e.offset:e.end]
                seg.copy_(sd.arrays[e.spec.name].reshape(-1).to(torch.float32))
                leaf = seg.view(e.spec.shape).detach().requires_grad_(True)
                leaf.grad = self.flat_grads[e.offset:e.end].view(e.spec.shape)
                self.views[e.spec.name] = leaf
                sd.arrays[e.spec.name] = seg.view(e.spec.shape)     # the graph's stored value now aliases the flat buffer
        self.updater = MultiLayerUpdater(entries, self.flat_params, self.flat_grads)
        self.updater.shadow, self.updater.shadow_offsets = self.flat_shadow, self.shadow_offsets
        self.refresh_shadow()

    def refresh_shadow(self):
        if self.flat_shadow is None:
            return
        with torch.no_grad():
            for e, so in zip(self.entries, self.shadow_offsets):
                self.flat_shadow[so:so + e.spec.numel].copy_(self.flat_params[e.offset:e.end])

    def values(self):
        """Variable values handed to the graph for a training step."""
        if self.flat_shadow is None:
            return dict(self.views)
        out = {}
        for e, so in zip(self.entries, self.shadow_offsets):
            leaf = self.views[e.spec.name]
            sh = self.flat_shadow[so:so + e.spec.numel].view(e.spec.shape)
            t = _ShadowParam.apply(leaf, sh)
            t._master = leaf
            out[e.spec.name] = t
        return out

    def step(self, placeholders):
        from .session import InferenceSession
        sd, tc = self.sd, self.tc
        losses = sd.lossVariables or tc.lossVariables
        if not losses:
            raise ValueError("no loss variables: call sd.setLossVariables(...)")
        hook = self.gradient_hook
        if hook is not None and hasattr(hook, "pre_step"):
            hook.pre_step(tc.iterationCount, tc.epochCount)       # per-step device variables of an overlapped exchange
        def fwd_bwd(ph):
            vals = InferenceSession(sd).run(ph, losses, self.values(), training=True)
            loss = vals[losses[0]].sum() if len(losses) == 1 else sum(vals[l].sum() for l in losses)
            if not tc.minimize:
                loss = -loss
            loss.backward()
            if hook is not None and hasattr(hook, "after_backward"):
                hook.after_backward()                             # flush + join of the side stream (inside a graph capture too)
            return loss.detach()
        if tc.cudaGraphs and self.flat_params.is_cuda and not sd.listeners:
            self.score = self._graphed(placeholders, fwd_bwd)
        else:
            self.score = fwd_bwd(placeholders)
        with torch.no_grad():
            if not (self.gradient_hook is not None and self.gradient_hook(self) is True):
                self.updater.update(tc.iterationCount, tc.epochCount)
                if self.flat_shadow is not None and not self.updater._shadow_fresh:
                    self.refresh_shadow()
                if not getattr(self.updater, "_fused_zeroes_grads", False) or not self.flat_params.is_cuda:
                    self.flat_grads.zero_()
        tc.iterationCount += 1
        return self.score


    def _graphed(self, placeholders, fwd_bwd, warmup=1):
        """Forward + backward through a CUDA graph captured per placeholder signature (the updater stays outside, so
        schedules and the Adam step count keep working).  The first ``warmup`` steps of a signature run eagerly."""
        from ..ops import native
        from .core import _tensor
        dev = self.sd.device
        names = sorted(k.name if hasattr(k, "name") else k for k in placeholders)
        src = {(k.name if hasattr(k, "name") else k): v for k, v in placeholders.items()}
        tensors = [_tensor(src[n]) for n in names]          # host (pinned) tensors are copied straight into the static inputs
        key = tuple((n, tuple(t.shape), t.dtype) for n, t in zip(names, tensors))
        cache = self.__dict__.setdefault("_cg_entries", {})
        e = cache.setdefault(key, {"seen": 0, "graph": None})
        if e["graph"] is None:
            e["seen"] += 1
            if e["seen"] <= warmup:
                return fwd_bwd({n: (t if t.device == dev else t.to(dev, non_blocking=True)) for n, t in zip(names, tensors)})
            e["static"] = [t.to(dev, copy=True) for t in tensors]
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            n0 = native.LAUNCHES
            with torch.cuda.graph(g):
                loss = fwd_bwd(dict(zip(names, e["static"])))
            e["launches"] = native.LAUNCHES - n0
            native.LAUNCHES = n0
            e["loss"], e["graph"] = loss, g
        for dst, t in zip(e["static"], tensors):
            dst.copy_(t, non_blocking=True)
        e["graph"].replay()
        native.LAUNCHES += e["launches"]
        return e["loss"]


class History:
    """``autodiff/listeners/records/History.java``: per-iteration loss curve and epoch timings."""

    def __init__(self):
        self.losses, self.epochTimes, self.trainEvaluations, self.validationEvaluations = [], [], {}, {}

    def lossCurve(self):
        return self

    def meanLoss(self, epoch=-1):
        ls = self.losses[epoch]
        return sum(ls) / max(len(ls), 1)

    def finalTrainingEvaluations(self):
        return self.trainEvaluations


def _ensure_state(sd) -> TrainingState:
    if sd.trainingConfig is None:
        raise ValueError("setTrainingConfig(...) must be called before fit")
    if sd._training is None:
        sd._training = TrainingState(sd)
    return sd._training


def fit(sd, data=None, epochs=1, validationData=None, validationFrequency=1, listeners=None, record_losses=True):
    st = _ensure_state(sd)
    tc = sd.trainingConfig
    hist = History()
    ls = list(sd.listeners) + list(listeners or [])

    def fire(name, *a):
        for l in ls:
            fn = getattr(l, name, None)
            if fn is not None:
                fn(sd, *a)
    single = hasattr(data, "getFeatures") and not hasattr(data, "hasNext")
    if isinstance(data, dict):
        single = True
    for ep in range(epochs):
        fire("epochStart", tc.epochCount)
        t0 = time.perf_counter()
        ep_losses = []
        batches = [data] if single else data
        if not single and hasattr(data, "reset"):
            data.reset()
        for ds in batches:
            ph = ds if isinstance(ds, dict) else tc.placeholders_from(ds)
            loss = st.step(ph)
            if record_losses:
                ep_losses.append(loss)
            if ls:
                fire("iterationDone", tc.iterationCount - 1, tc.epochCount, loss)
        hist.losses.append([float(l) for l in ep_losses])
        hist.epochTimes.append(time.perf_counter() - t0)
        tc.epochCount += 1
        fire("epochEnd", tc.epochCount - 1)
        if validationData is not None and (ep + 1) % validationFrequency == 0 and tc.validationEvaluations:
            for var, (idx, evals) in tc.validationEvaluations.items():
                sd.evaluate(validationData, var, *evals)
                hist.validationEvaluations[var] = evals
    return hist
