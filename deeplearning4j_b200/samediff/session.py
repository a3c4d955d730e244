"""Graph execution (``InferenceSession`` / ``TrainingSession``).

Parity: ``nd4j-api/.../autodiff/samediff/internal/AbstractSession.java:161-935`` (dependency-driven
execution of the sub-graph needed for the requested outputs) and ``InferenceSession.doExec``
``:1373``.  Nodes are stored in creation order, which is already a valid schedule, so the session
filters that list to the ancestors of the requested outputs, applies the graph-optimizer fusions
(``autodiff/samediff/optimize``: here ``xw_plus_b -> gelu`` becomes one fused GEMM-epilogue node)
and runs it.  The plan is cached per (outputs, training) pair.
"""
from __future__ import annotations

import torch

from ..ops import registry
from .core import SameDiffOp, VariableType, _tensor

_TRAINING_AWARE = {"dropout", "dropout_inverted", "dot_product_attention_v2", "alpha_dropout"}


class ExecutionPlan:
    def __init__(self, nodes, fused):
        self.nodes = nodes      # list of (node, opdef, fused_with)
        self.fused = fused


def _build_plan(sd, outputs):
    nodes = sd._needed_ops(outputs)
    consumers = {}
    for n in nodes:
        for i in n.inputs:
            if i is not None:
                consumers.setdefault(i, []).append(n)
    out_set = set(outputs)
    skip, plan = set(), []
    for n in nodes:
        if id(n) in skip:
            continue
        # fusion: xw_plus_b whose only consumer is a gelu node
        if n.opName in ("xw_plus_b", "linear") and len(n.outputs) == 1 and n.outputs[0] not in out_set \
                and not n.args.get("transposeW") and not n.args.get("aTranspose"):
            cs = consumers.get(n.outputs[0], [])
            if len(cs) == 1 and cs[0].opName in ("gelu", "precise_gelu") and len(cs[0].inputs) == 1:
                g = cs[0]
                fused = SameDiffOp(n.name, "linear_gelu", list(n.inputs), list(g.outputs), {"precise": g.opName == "precise_gelu"})
                plan.append((fused, registry.get("linear_gelu")))
                skip.add(id(g))
                continue
        plan.append((n, registry.get(n.opName)))
    return plan


class InferenceSession:
    def __init__(self, sd):
        self.sd = sd

    def run(self, placeholders, outputs, values=None, training=False):
        sd = self.sd
        outputs = list(outputs)
        key = (tuple(outputs), bool(training))
        if sd._exec_plan is None:
            sd._exec_plan = {}
        plan = sd._exec_plan.get(key)
        if plan is None:
            plan = _build_plan(sd, outputs)
            sd._exec_plan[key] = plan
        vals = dict(values) if values else {}
        dev = sd.device
        for k, v in (placeholders or {}).items():
            k = k.name if hasattr(k, "name") else k
            if k not in vals:
                t = _tensor(v)
                vals[k] = t if t.device == dev else t.to(dev, non_blocking=True)
        arrays = sd.arrays
        listeners = sd.listeners
        for node, d in plan:
            ins = []
            for i in node.inputs:
                if i is None:
                    ins.append(None)
                    continue
                v = vals.get(i)
                if v is None:
                    v = arrays.get(i)
                    if v is None:
                        var = sd.variables.get(i)
                        if var is not None and var.variableType == VariableType.PLACEHOLDER:
                            raise ValueError(f"no value provided for placeholder '{i}' required by op '{node.name}'")
                        raise ValueError(f"variable '{i}' has no value (op '{node.name}')")
                ins.append(v)
            args = node.args
            if listeners:
                for l in listeners:
                    fn = getattr(l, "preOpExecution", None)
                    if fn is not None:
                        fn(sd, node)
            if node.opName == "while_loop":
                res = _run_while(sd, ins, args["body"], vals)
            elif d.group == "random" and not ins and "shape" in args:
                res = d.fn(device=dev, **args)
            elif node.opName in _TRAINING_AWARE:
                res = d.fn(*ins, training=training, **args)
            else:
                res = d.fn(*ins, **args)
            outs = node.outputs
            if isinstance(res, (tuple, list)) and not (len(outs) == 1 and d.n_out == 1):
                for o, r in zip(outs, res):
                    vals[o] = r
            else:
                vals[outs[0]] = res
            if listeners:
                for l in listeners:
                    fn = getattr(l, "opExecution", None)
                    if fn is not None:
                        fn(sd, node, [vals[o] for o in outs if o in vals])
        for o in outputs:
            if o not in vals:
                if o in arrays:
                    vals[o] = arrays[o]
                else:
                    raise ValueError(f"requested output '{o}' was not produced")
        return vals


def _run_while(sd, ins, body, vals):
    """Eager loop: ``cond_fn`` / ``body_fn`` receive and return torch tensors."""
    _, cond_fn, body_fn, n = body
    state = list(ins)
    it = 0
    while bool(torch.as_tensor(cond_fn(*state)).all()):
        r = body_fn(*state)
        state = list(r) if isinstance(r, (list, tuple)) else [r]
        it += 1
        if it > 10_000_000:
            raise RuntimeError("whileLoop exceeded 1e7 iterations")
    return tuple(state)


registry.op("while_loop", n_out=-1)(lambda *a, **kw: a)
