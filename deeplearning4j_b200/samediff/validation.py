"""SameDiff validation utilities (``nd4j-api/.../autodiff/validation``): ``GradCheckUtil`` (numerical vs autograd
gradients of a graph's loss), ``OpTestCase`` / ``TestCase`` with expected outputs, and ``OpValidation`` which also
keeps the op-coverage bookkeeping the reference prints at the end of its test run."""
from __future__ import annotations

import torch

from ..nd.ndarray import INDArray
from ..ops import registry


def _t(x):
    return x.t if isinstance(x, INDArray) else (x if isinstance(x, torch.Tensor) else torch.as_tensor(x))


class GradCheckUtil:
    DEFAULT_EPS = 1e-5
    DEFAULT_MAX_REL_ERROR = 1e-5
    DEFAULT_MIN_ABS_ERROR = 1e-6

    @staticmethod
    def checkGradients(sd, placeholders=None, eps=DEFAULT_EPS, maxRelError=DEFAULT_MAX_REL_ERROR, minAbsError=DEFAULT_MIN_ABS_ERROR,
                       print_=False, exitOnFirstFailure=False, skipVariables=(), maxPerParam=50, seed=12345):
        """Central differences on every trainable variable (in float64) against ``calculateGradients``."""
        from .core import VariableType
        if not sd.lossVariables:
            raise ValueError("Expected 1 or more loss function variables for gradient check, got 0")
        ph = {k: _t(v).double() if _t(v).is_floating_point() else _t(v) for k, v in (placeholders or {}).items()}
        saved = dict(sd.arrays)
        names = [v.name for v in sd.trainableVariables() if v.name not in skipVariables]
        try:
            for n in list(sd.arrays):
                if sd.arrays[n].is_floating_point():
                    sd.arrays[n] = sd.arrays[n].detach().double().clone()
            sd._exec_plan = None
            grads = sd.calculateGradients(ph, *names)
            gen = torch.Generator().manual_seed(seed)
            fails, total = [], 0

            def loss():
                out = sd.output(ph, *sd.lossVariables)
                return float(sum(_t(out[l]).double().sum() for l in sd.lossVariables))
            for n in names:
                arr = sd.arrays[n]
                flat = arr.reshape(-1)
                g = _t(grads[n]).reshape(-1)
                idx = torch.randperm(flat.numel(), generator=gen)[:maxPerParam].tolist()
                for i in idx:
                    o = float(flat[i])
                    flat[i] = o + eps
                    lp = loss()
                    flat[i] = o - eps
                    lm = loss()
                    flat[i] = o
                    num, ana = (lp - lm) / (2 * eps), float(g[i])
                    den = abs(num) + abs(ana)
                    rel = abs(num - ana) / den if den > 0 else 0.0
                    total += 1
                    if rel > maxRelError and abs(num - ana) > minAbsError:
                        fails.append((n, i, ana, num, rel))
                        if print_:
                            print(f"{n}[{i}] FAILED: analytic={ana:.8g} numerical={num:.8g} relError={rel:.3g}")
                        if exitOnFirstFailure:
                            return False
            if print_:
                print(f"GradCheckUtil: {total} checked, {len(fails)} failed")
            return not fails
        finally:
            sd.arrays.clear()
            sd.arrays.update(saved)
            sd._exec_plan = None


class TestCase:
    """A SameDiff graph + placeholder values + expected outputs (+ optional gradient check)."""
    __test__ = False

    def __init__(self, sd):
        self.sd, self.expected, self.placeholders = sd, {}, {}
        self.gradientCheck_, self.testName_ = True, None
        self.maxRelError, self.minAbsError, self.eps = 1e-5, 1e-6, 1e-5
        self.skip = ()

    def testName(self, n): self.testName_ = n; return self
    def expected_(self, var, arr): self.expected[getattr(var, "name", var)] = arr; return self
    expectedOutput = expected_
    def placeholderValue(self, name, arr): self.placeholders[name] = arr; return self
    def placeholderValues(self, m): self.placeholders.update(m); return self
    def gradientCheck(self, b): self.gradientCheck_ = b; return self
    def gradCheckSkipVariables(self, *n): self.skip = n; return self
    def gradCheckMaxRelativeError(self, v): self.maxRelError = v; return self
    def gradCheckMinAbsError(self, v): self.minAbsError = v; return self
    def gradCheckEpsilon(self, v): self.eps = v; return self


class OpTestCase:
    """Single-op check: expected output arrays (or predicates) and optionally expected shapes."""
    def __init__(self, opName, inputs=(), **args):
        self.opName, self.inputs, self.args = opName, list(inputs), args
        self.expected, self.shapes = {}, {}
    def expectedOutput(self, idx, arr, eps=1e-5): self.expected[idx] = (arr, eps); return self
    def expectedOutputShape(self, idx, shape): self.shapes[idx] = tuple(shape); return self


class OpValidation:
    _executed = set()
    _validated = set()

    @staticmethod
    def validate(tc):
        """Returns None when the test case passes, otherwise an error string (as the reference does)."""
        if isinstance(tc, OpTestCase):
            OpValidation._executed.add(tc.opName)
            out = registry.get(tc.opName).fn(*[_t(i) if i is not None else None for i in tc.inputs], **tc.args)
            outs = list(out) if isinstance(out, (tuple, list)) else [out]
            for i, shp in tc.shapes.items():
                if tuple(outs[i].shape) != shp:
                    return f"{tc.opName}: output {i} shape {tuple(outs[i].shape)} != expected {shp}"
            for i, (exp, eps) in tc.expected.items():
                if callable(exp):
                    r = exp(outs[i])
                    if r not in (None, True):
                        return f"{tc.opName}: output {i} failed predicate: {r}"
                    continue
                e = _t(exp)
                if tuple(e.shape) != tuple(outs[i].shape):
                    return f"{tc.opName}: output {i} shape {tuple(outs[i].shape)} != expected {tuple(e.shape)}"
                if not torch.allclose(outs[i].double(), e.double().to(outs[i].device), atol=eps, rtol=eps, equal_nan=True):
                    return f"{tc.opName}: output {i} differs from expected (max abs err {float((outs[i].double() - e.double()).abs().max()):.3g})"
            OpValidation._validated.add(tc.opName)
            return None
        sd = tc.sd
        for op in sd.ops:
            OpValidation._executed.add(op.opName)
        if tc.expected:
            out = sd.output(tc.placeholders, *tc.expected)
            for n, exp in tc.expected.items():
                got = _t(out[n])
                if callable(exp):
                    r = exp(got)
                    if r not in (None, True):
                        return f"{tc.testName_ or ''}: variable {n} failed predicate: {r}"
                    continue
                e = _t(exp).to(got.device)
                if tuple(e.shape) != tuple(got.shape):
                    return f"{tc.testName_ or ''}: variable {n} shape {tuple(got.shape)} != expected {tuple(e.shape)}"
                if not torch.allclose(got.double(), e.double(), atol=1e-5, rtol=1e-5, equal_nan=True):
                    return f"{tc.testName_ or ''}: variable {n} differs from expected"
        if tc.gradientCheck_ and sd.lossVariables:
            if not GradCheckUtil.checkGradients(sd, tc.placeholders, tc.eps, tc.maxRelError, tc.minAbsError, skipVariables=tc.skip):
                return f"{tc.testName_ or ''}: gradient check failed"
        for op in sd.ops:
            OpValidation._validated.add(op.opName)
        return None

    @staticmethod
    def coverage():
        names = set(registry.names())
        return {"total": len(names), "executed": len(OpValidation._executed & names), "validated": len(OpValidation._validated & names),
                "notValidated": sorted(names - OpValidation._validated)}

    @staticmethod
    def logCoverageInformation(logUnvalidated=False):
        c = OpValidation.coverage()
        lines = [f"Op validation coverage: {c['validated']}/{c['total']} validated, {c['executed']} executed"]
        if logUnvalidated:
            lines += ["  not validated: " + ", ".join(c["notValidated"])]
        return "\n".join(lines)
