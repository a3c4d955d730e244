"""Graph execution (``InferenceSession`` / ``TrainingSession``).

Parity: ``nd4j-api/.../autodiff/samediff/internal/AbstractSession.java:161-935`` (dependency-driven
execution of the sub-graph needed for the requested outputs) and ``InferenceSession.doExec``
``:1373``.  Nodes are stored in creation order, which is already a valid schedule, so the session
filters that list to the ancestors of the requested outputs, applies the graph-optimizer fusions
(``autodiff/samediff/optimize``: here ``xw_plus_b -> gelu`` becomes one fused GEMM-epilogue node)
and runs it.  The plan is cached per (outputs, training) pair.
"""
from __future__ import annotations

import os

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
    # fusion: add whose only consumer is a layer_norm taking it as its input (residual connection + norm); the fused node sits at
    # the layer_norm's position, where the gain / bias inputs are certainly available
    fuse_ln, fuse_mlp = {}, {}
    for n in nodes:
        if n.opName == "add" and len(n.inputs) == 2 and None not in n.inputs and len(n.outputs) == 1 and n.outputs[0] not in out_set:
            cs = consumers.get(n.outputs[0], [])
            if len(cs) == 1 and cs[0].opName == "layer_norm" and cs[0].inputs and cs[0].inputs[0] == n.outputs[0] \
                    and cs[0].inputs.count(n.outputs[0]) == 1:
                ln = cs[0]
                fuse_ln[id(ln)] = SameDiffOp(ln.name, "add_layer_norm", list(n.inputs) + list(ln.inputs[1:]), list(ln.outputs), dict(ln.args))
                skip.add(id(n))
    for n in nodes:
        if id(n) in skip:
            continue
        if id(n) in fuse_ln:
            plan.append((fuse_ln[id(n)], registry.get("add_layer_norm")))
            continue
        if id(n) in fuse_mlp:
            plan.append((fuse_mlp[id(n)], registry.get("mlp_gelu")))
            continue
        # fusion: xw_plus_b whose only consumer is a gelu node
        if n.opName in ("xw_plus_b", "linear") and len(n.outputs) == 1 and n.outputs[0] not in out_set \
                and not n.args.get("transposeW") and not n.args.get("aTranspose"):
            cs = consumers.get(n.outputs[0], [])
            if len(cs) == 1 and cs[0].opName in ("gelu", "precise_gelu") and len(cs[0].inputs) == 1:
                g = cs[0]
                # ... and a second linear layer as the gelu's only consumer: the whole feed-forward block can be one node, placed where
                # the second layer stood (its weights are certainly available there).  Off unless DL4J_FUSE_MLP=1: measured on
                # BERT-base the step got slower (19.98 against 15.91 ms), because the data-gradient GEMM's epilogue fetches the
                # pre-activations with per-thread row loads whose latency it cannot hide, which costs more than the saved pass.
                cs2 = consumers.get(g.outputs[0], []) if len(g.outputs) == 1 and g.outputs[0] not in out_set else []
                m = cs2[0] if len(cs2) == 1 else None
                if m is not None and m.opName in ("xw_plus_b", "linear") and m.inputs and m.inputs[0] == g.outputs[0] \
                        and m.inputs.count(g.outputs[0]) == 1 and not m.args.get("transposeW") and not m.args.get("aTranspose") \
                        and len(n.inputs) == 3 and len(m.inputs) in (2, 3) and os.environ.get("DL4J_FUSE_MLP", "0") == "1":
                    fuse_mlp[id(m)] = SameDiffOp(m.name, "mlp_gelu", list(n.inputs) + list(m.inputs[1:]), list(m.outputs),
                                                 {"precise": g.opName == "precise_gelu"})
                    skip.add(id(g))
                    continue
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
        logic = sd._exec_plan.get("__logic__")
        if logic is None:
            from .controlflow import has_logic_ops
            logic = sd._exec_plan["__logic__"] = has_logic_ops(sd)
        if logic:
            # graphs with enter / exit / switch / merge / next_iteration nodes have cycles: the frame-aware executor runs them
            from .controlflow import DataflowExecutor
            vals = DataflowExecutor(sd, training).run(placeholders, values)
            for o in outputs:
                if o not in vals:
                    raise ValueError(f"requested output '{o}' was not produced (its branch was not taken, or an input is missing)")
            return vals
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


def _exec_ops(sd, ops, local, training=False):
    """Run a captured op list (loop condition / body) over ``local`` values, falling back to the graph's arrays."""
    for node in ops:
        d = registry.get(node.opName)
        ins = []
        for i in node.inputs:
            if i is None:
                ins.append(None)
                continue
            v = local.get(i)
            if v is None:
                v = sd.arrays.get(i)
            if v is None:
                raise ValueError(f"variable '{i}' has no value inside loop op '{node.name}'")
            ins.append(v)
        if node.opName == "while_loop":
            res = _run_while(sd, ins, node.args["body"], local)
        elif node.opName in _TRAINING_AWARE:
            res = d.fn(*ins, training=training, **node.args)
        else:
            res = d.fn(*ins, **node.args)
        if isinstance(res, (tuple, list)) and not (len(node.outputs) == 1 and d.n_out == 1):
            for o, r in zip(node.outputs, res):
                local[o] = r
        else:
            local[node.outputs[0]] = res


def _run_while(sd, ins, body, vals):
    """Eager loop.  Two body forms: Python callables over torch tensors, or op lists captured from SameDiff
    lambdas (``SameDiff.whileLoop``), whose loop-carried inputs are fed through stand-in variables."""
    if body[0] == "graph":
        _, ph_names, cond_name, cond_ops, out_names, body_ops, extra_names = body
        n = len(ph_names)
        state = list(ins[:n])
        outer = dict(zip(extra_names, ins[n:]))
        it = 0
        while True:
            local = dict(outer)
            local.update(zip(ph_names, state))
            _exec_ops(sd, cond_ops, local)
            if not bool(torch.as_tensor(local[cond_name]).all()):
                break
            _exec_ops(sd, body_ops, local)
            state = [local[o] for o in out_names]
            it += 1
            if it > 10_000_000:
                raise RuntimeError("whileLoop exceeded 1e7 iterations")
        return tuple(state)
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
