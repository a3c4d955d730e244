"""``GradientCheckUtil`` (``deeplearning4j-nn/.../gradientcheck/GradientCheckUtil.java``): central-difference
check of the analytic gradients of a MultiLayerNetwork / ComputationGraph against the score function, in
double precision, parameter by parameter (or a random subset)."""
from __future__ import annotations

import random

import torch


class GradientCheckUtil:
    DEFAULT_EPS = 1e-6
    DEFAULT_MAX_REL_ERROR = 1e-3
    DEFAULT_MIN_ABS_ERROR = 1e-8

    @staticmethod
    def _to_double(net):
        """A float64 copy of the network (the reference requires DOUBLE data type for gradient checks)."""
        from ..nd.dtype import DataType
        conf = net.conf.clone()
        conf.dataType = DataType.DOUBLE
        conf.computeDataType = None
        m = type(net)(conf)
        m.device = net.device
        p = net.params()
        p = p.t if hasattr(p, "t") and not isinstance(p, torch.Tensor) else p
        m.init(p.double(), True)
        return m

    @staticmethod
    def checkGradients(net, input=None, labels=None, epsilon=DEFAULT_EPS, maxRelError=DEFAULT_MAX_REL_ERROR, minAbsoluteError=DEFAULT_MIN_ABS_ERROR,
                       print_=False, exitOnFirstError=False, inputMask=None, labelMask=None, subset=False, maxPerParam=None, seed=12345,
                       excludeParams=None, returnDetails=False):
        if hasattr(input, "getFeatures"):
            ds = input
            input, labels, inputMask, labelMask = ds.getFeatures(), ds.getLabels(), ds.getFeaturesMaskArray(), ds.getLabelsMaskArray()
        from .updaters import NoOp, Sgd
        for e in net.entries:
            u = e.layer.updater_for(e.spec) if hasattr(e.layer, "updater_for") else None
            if u is not None and not isinstance(u, (NoOp, Sgd)):
                pass                                              # the updater is never applied here; only the raw gradient is used
        dbl = GradientCheckUtil._to_double(net)
        as_d = lambda t: None if t is None else (t.t if hasattr(t, "t") and not isinstance(t, torch.Tensor) else torch.as_tensor(t)).double()
        as_in = lambda v: [as_d(x) for x in v] if isinstance(v, (list, tuple)) else as_d(v)
        x, y, fm, lm = as_in(input), as_in(labels), as_in(inputMask), as_in(labelMask)

        from ..data.dataset import DataSet, MultiDataSet
        multi = isinstance(x, list)
        ds = MultiDataSet(x, y if isinstance(y, list) else [y], fm, lm) if multi else DataSet(x, y, fm, lm)

        def score():
            # data term only: regularisation is applied by the updater and is not part of the raw gradient
            reg = dbl._regularization_score()
            return dbl._score_dataset(ds, True) - (float(reg) if reg is not None else 0.0)

        dbl.flat_grads.zero_()
        dbl.computeGradientAndScore(x, y, fm, lm)
        analytic = dbl.flat_grads.clone()
        params = dbl.flat_params
        rng = random.Random(seed)
        fails, checked, worst = [], 0, 0.0
        for e in dbl.entries:
            if e.spec.kind == "state" or (excludeParams and e.key in excludeParams):
                continue
            idxs = list(range(e.offset, e.end))
            if subset and maxPerParam and len(idxs) > maxPerParam:
                idxs = rng.sample(idxs, maxPerParam)
            for i in idxs:
                orig = float(params[i])
                params[i] = orig + epsilon
                sp = score()
                params[i] = orig - epsilon
                sm = score()
                params[i] = orig
                numeric = (sp - sm) / (2 * epsilon)
                a = float(analytic[i])
                denom = abs(a) + abs(numeric)
                rel = abs(a - numeric) / denom if denom > 0 else 0.0
                checked += 1
                if rel > maxRelError and abs(a - numeric) > minAbsoluteError:
                    fails.append((e.key, i - e.offset, a, numeric, rel))
                    if print_:
                        print(f"Param {e.key}[{i - e.offset}] FAILED: grad={a:.8g}, numericalGrad={numeric:.8g}, relError={rel:.4g}")
                    if exitOnFirstError:
                        return (False, fails, checked) if returnDetails else False
                worst = max(worst, rel if abs(a - numeric) > minAbsoluteError else 0.0)
        if print_:
            print(f"GradientCheckUtil.checkGradients(): {checked} params checked, {checked - len(fails)} passed, {len(fails)} failed. Largest relative error = {worst:.4g}")
        ok = not fails
        return (ok, fails, checked) if returnDetails else ok
