"""Graph-level control flow: Enter / Exit / Switch / Merge / NextIteration / LoopCond nodes, how ``ifCond`` / ``whileLoop``
emit them, and the frame-aware executor that runs them.

Parity: ``nd4j-api/.../autodiff/samediff/ControlFlow.java:139`` (``ifCond``) and ``:505`` (``whileLoop``) build these nodes, the
native executor runs them (``libnd4j/include/graph/execution/impl/Logic{Enter,Exit,Switch,Merge,NextIteration,LoopCond}.cpp``,
``graph/impl/GraphExecutioner.cpp:197,481``), and the Java session tracks ``(frame, iteration)`` per value
(``autodiff/samediff/internal/AbstractSession.java:161-935``).  Because the constructs are ordinary nodes they survive
``.fb`` save / load and are what TensorFlow-imported graphs contain.

Execution model (tagged-token dataflow).  Every value carries a tag: the stack of ``(frame name, iteration)`` pairs it lives in;
``()`` is the top level.  A node instance ``(node, tag)`` fires when its inputs with that tag have arrived.

* ``switch(x, pred)`` -> ``[false branch, true branch]``: the branch not taken receives a *dead* token; every ordinary node that
  sees a dead input emits dead outputs without computing anything, which is how the untaken branch of a conditional stays idle.
* ``merge(a, b, ..)`` forwards the first live input it receives (dead only when all inputs are dead).
* ``enter(x, frameName=f)``: tag ``T`` -> ``T + ((f, 0),)``; with ``isConstant`` the value is re-issued at every iteration of the frame.
* ``next_iteration(x)``: ``T + ((f, i),)`` -> ``T + ((f, i + 1),)``; dead tokens stop here (that is what ends a loop).
* ``exit(x)``: ``T + ((f, i),)`` -> ``T``; dead tokens are dropped.
* ``loop_cond(p)`` is the identity.

Tensors flow through torch, so a loop or a conditional is differentiable the usual way: autograd records whatever was executed.
"""
from __future__ import annotations

import torch

from ..ops import registry
from ..ops.registry import op

LOGIC_OPS = ("switch", "merge", "enter", "exit", "next_iteration", "loop_cond")
MAX_ITERATIONS = 10_000_000


class _Dead:
    def __repr__(self):
        return "<dead>"


DEAD = _Dead()

# the logic ops are executed by the executor itself; the registry entries make the names resolvable (op hashes, op listings)
op("switch", n_out=2, group="logic", differentiable=False)(lambda x, pred, **kw: (x, x))
op("enter", group="logic")(lambda x, **kw: x)
op("exit", group="logic")(lambda x, **kw: x)
op("next_iteration", group="logic")(lambda x, **kw: x)
op("loop_cond", group="logic", differentiable=False)(lambda x, **kw: x)
# ``depend(x, anchor) -> x``: ties a value to the frame and iteration of ``anchor`` (a loop built inside another loop's body enters
# from there even when the entering value was computed from constants only)
op("depend", group="logic")(lambda x, anchor=None, **kw: x)


def has_logic_ops(sd) -> bool:
    return any(o.opName in LOGIC_OPS for o in sd.ops)


def _truth(v) -> bool:
    return bool(torch.as_tensor(v).reshape(-1)[0]) if not isinstance(v, bool) else v


class DataflowExecutor:
    """Runs a graph that contains logic nodes.  ``run`` returns the top-level value of every variable that received one."""

    def __init__(self, sd, training=False, max_steps=200_000_000):
        self.sd, self.training, self.max_steps = sd, training, int(max_steps)
        self.consumers = {}
        for node in sd.ops:
            for k, i in enumerate(node.inputs):
                if i is not None:
                    self.consumers.setdefault(i, []).append((node, k))
        self.frame_of_enter = {n.name: n.args.get("frameName", n.name) for n in sd.ops if n.opName == "enter"}

    # ---------------------------------------------------------------------------------------------------------------
    def run(self, placeholders, values=None):
        from .core import VariableType, _tensor
        sd = self.sd
        dev = sd.device
        base = dict(values) if values else {}
        for k, v in (placeholders or {}).items():
            k = k.name if hasattr(k, "name") else k
            if k not in base:
                t = _tensor(v)
                base[k] = t if t.device == dev else t.to(dev)
        leaf = {}
        for name, var in sd.variables.items():
            if var.variableType in (VariableType.VARIABLE, VariableType.CONSTANT, VariableType.PLACEHOLDER):
                if name in base:
                    leaf[name] = base[name]
                elif name in sd.arrays:
                    leaf[name] = sd.arrays[name]
        self.leaf = leaf
        self.tokens = {}            # (variable, tag) -> value | DEAD
        self.fired = set()          # (node name, tag)
        self.constants = {}         # (frame path tuple) -> list of (enter node, value): re-issued every iteration
        self.iterations = {}        # frame path -> highest iteration started
        self.queue = []
        self.waiting = {}           # node name -> tags at which it was tried before all of its inputs had arrived
        # seeds: every node whose inputs are all leaves (or that has none) is ready at the top level
        for node in sd.ops:
            if all(i is None or i in leaf for i in node.inputs):
                self.queue.append((node, ()))
        steps = 0
        while self.queue:
            node, tag = self.queue.pop()
            self._try_fire(node, tag)
            steps += 1
            if steps > self.max_steps:
                raise RuntimeError(f"control-flow execution did not finish within {self.max_steps} node firings")
        out = dict(leaf)
        for (name, tag), v in self.tokens.items():
            if tag == () and v is not DEAD:
                out[name] = v
        return out

    # ---------------------------------------------------------------------------------------------------------------
    def _value(self, name, tag):
        """Value of ``name`` visible at ``tag``: a token with that tag, else a leaf (leaves are visible everywhere)."""
        if name in self.leaf:
            return self.leaf[name]
        # a value of an enclosing frame (same iteration of that frame) is visible inside the frames nested in it; graphs written
        # by TensorFlow route such reads through constant ``enter`` nodes, hand-built ones need not
        for k in range(len(tag), -1, -1):
            v = self.tokens.get((name, tag[:k]))
            if v is not None:
                return v
        return None

    def _emit(self, name, tag, value):
        key = (name, tag)
        if key in self.tokens:
            return
        self.tokens[key] = value
        n = len(tag)
        for node, _ in self.consumers.get(name, ()):
            self.queue.append((node, tag))
            for wt in self.waiting.get(node.name, ()):
                if len(wt) > n and wt[:n] == tag:
                    self.queue.append((node, wt))

    def _try_fire(self, node, tag):
        key = (node.name, tag)
        if key in self.fired:
            return
        opn = node.opName
        if opn == "merge":
            vals = [self._value(i, tag) for i in node.inputs if i is not None]
            live = [v for v in vals if v is not None and v is not DEAD]
            if live:
                self.fired.add(key)
                self._emit(node.outputs[0], tag, live[0])
            elif vals and all(v is DEAD for v in vals):
                self.fired.add(key)
                self._emit(node.outputs[0], tag, DEAD)
            return
        ins = []
        for i in node.inputs:
            if i is None:
                ins.append(None)
                continue
            v = self._value(i, tag)
            if v is None:
                self.waiting.setdefault(node.name, set()).add(tag)
                return                      # not ready
            ins.append(v)
        self.fired.add(key)
        dead = any(v is DEAD for v in ins)
        if opn == "enter":
            frame = node.args.get("frameName", node.name)
            new_tag = tag + ((frame, 0),)
            if dead:
                self._emit(node.outputs[0], new_tag, DEAD)
                return
            if node.args.get("isConstant"):
                path = tag + (frame,)
                self.constants.setdefault(path, []).append((node, ins[0]))
                for it in range(self.iterations.get(path, 0) + 1):
                    self._emit(node.outputs[0], tag + ((frame, it),), ins[0])
            else:
                self._emit(node.outputs[0], new_tag, ins[0])
            return
        if opn == "exit":
            if not dead and tag:
                self._emit(node.outputs[0], tag[:-1], ins[0])
            elif not tag:
                self._emit(node.outputs[0], tag, ins[0])
            return
        if opn == "next_iteration":
            if dead or not tag:
                return
            frame, it = tag[-1]
            if it + 1 > MAX_ITERATIONS:
                raise RuntimeError(f"loop '{frame}' exceeded {MAX_ITERATIONS} iterations")
            new_tag = tag[:-1] + ((frame, it + 1),)
            path = tag[:-1] + (frame,)
            if self.iterations.get(path, 0) < it + 1:
                self.iterations[path] = it + 1
                for enter_node, val in self.constants.get(path, ()):          # loop invariants follow into the new iteration
                    self._emit(enter_node.outputs[0], new_tag, val)
            self._emit(node.outputs[0], new_tag, ins[0])
            return
        if opn == "switch":
            if dead:
                for o in node.outputs:
                    self._emit(o, tag, DEAD)
                return
            taken = _truth(ins[1])
            self._emit(node.outputs[0], tag, DEAD if taken else ins[0])        # output 0: predicate false
            if len(node.outputs) > 1:
                self._emit(node.outputs[1], tag, ins[0] if taken else DEAD)    # output 1: predicate true
            return
        if dead:
            for o in node.outputs:
                self._emit(o, tag, DEAD)
            return
        if opn == "loop_cond":
            self._emit(node.outputs[0], tag, ins[0])
            return
        d = registry.get(opn)
        if opn in ("dropout", "dropout_inverted", "dot_product_attention_v2", "alpha_dropout"):
            res = d.fn(*ins, training=self.training, **node.args)
        else:
            res = d.fn(*ins, **node.args)
        outs = node.outputs
        if isinstance(res, (tuple, list)) and not (len(outs) == 1 and d.n_out == 1):
            for o, r in zip(outs, res):
                self._emit(o, tag, r)
            for o in outs[len(res):]:
                self._emit(o, tag, res[-1] if len(res) else DEAD)
        else:
            self._emit(outs[0], tag, res)
            for o in outs[1:]:
                self._emit(o, tag, res)


# ----------------------------------------------------------------------------------------------------- graph construction
def _outer_reads(sd, first_op, produced_inside):
    """Names read by the ops added since ``first_op`` that were produced outside of them (and are not leaves)."""
    from .core import VariableType
    reads = []
    for node in sd.ops[first_op:]:
        for i in node.inputs:
            if i is None or i in produced_inside or i in reads:
                continue
            var = sd.variables.get(i)
            if var is not None and var.variableType == VariableType.ARRAY:
                reads.append(i)
    return reads


def _rewire(sd, first_op, mapping):
    for node in sd.ops[first_op:]:
        node.inputs = [mapping.get(i, i) if i is not None else None for i in node.inputs]


def build_if(sd, cond_fn, true_fn, false_fn, name=None):
    """``ifCond``: ``pred = cond(sd)``; both branch lambdas are traced into the graph; every outer array a branch reads is routed
    through a ``switch`` on the predicate (so only the taken branch computes), and the results meet in a ``merge``."""
    base = name or sd._unique("cond")
    pred = cond_fn(sd)
    pred = sd._op("identity", [pred], name=f"{base}/pred_id")
    outs = []
    for branch, fn, port in (("truefn", true_fn, 1), ("falsefn", false_fn, 0)):
        first = len(sd.ops)
        n_vars = set(sd.variables)
        r = fn(sd)
        produced = set(sd.variables) - n_vars
        reads = _outer_reads(sd, first, produced)
        mapping = {}
        body_ops = sd.ops[first:]
        del sd.ops[first:]
        for rname in reads:
            sw = sd._op("switch", [sd.variables[rname], pred], name=f"{base}/{branch}/Switch", frameName=base)
            mapping[rname] = sw[port].name
        sd.ops.extend(body_ops)
        for node in body_ops:
            node.inputs = [mapping.get(i, i) if i is not None else None for i in node.inputs]
        rn = r.name if hasattr(r, "name") else r
        if rn in mapping:
            rn = mapping[rn]
        elif rn not in produced:
            # a branch that returns a leaf (or computes nothing): gate it so that the merge sees exactly one live input
            sw = sd._op("switch", [sd.variables[rn], pred], name=f"{base}/{branch}/Switch", frameName=base)
            rn = sw[port].name
        elif not reads:
            # a branch made only of leaves and constants still has to be dead when not taken
            sw = sd._op("switch", [sd.variables[rn], pred], name=f"{base}/{branch}/Switch", frameName=base)
            rn = sw[port].name
        outs.append(sd.variables[rn])
    sd._exec_plan = None
    return sd._op("merge", [outs[1], outs[0]], name=f"{base}/Merge" if name is None else name, frameName=base)


def build_while(sd, loop_vars, cond_fn, body_fn, name=None):
    """``whileLoop``: the TensorFlow-style frame ``enter -> merge -> cond -> loop_cond -> switch -> (exit | body -> next_iteration)``;
    arrays of the enclosing scope that the condition or the body read come in through constant ``enter`` nodes."""
    frame = name or sd._unique("while")
    n = len(loop_vars)
    anchors = sd.__dict__.setdefault("_cf_anchors", [])
    anchor = anchors[-1] if anchors else None

    def anchored(v):
        return v if anchor is None else sd._op("depend", [v, anchor], name=f"{frame}/Depend")
    enters = [sd._op("enter", [anchored(v)], name=f"{frame}/Enter", frameName=frame, isConstant=False) for v in loop_vars]
    merges = []
    merge_nodes = []
    for e in enters:
        m = sd._op("merge", [e, e], name=f"{frame}/Merge", frameName=frame)      # second input patched to next_iteration below
        merges.append(m)
        merge_nodes.append(sd._producer[m.name])
    first_cond = len(sd.ops)
    before = set(sd.variables)
    pred = cond_fn(sd, list(merges))
    cond_produced = set(sd.variables) - before
    lc = sd._op("loop_cond", [pred], name=f"{frame}/LoopCond", frameName=frame)
    switches = [sd._op("switch", [m, lc], name=f"{frame}/Switch", frameName=frame) for m in merges]
    exits = [sd._op("exit", [s[0]], name=f"{frame}/Exit", frameName=frame) for s in switches]
    idents = [sd._op("identity", [s[1]], name=f"{frame}/Identity") for s in switches]
    before = set(sd.variables)
    anchors.append(idents[0])            # loops built inside this body enter from this frame's current iteration
    try:
        r = body_fn(sd, list(idents))
    finally:
        anchors.pop()
    r = list(r) if isinstance(r, (list, tuple)) else [r]
    if len(r) != n:
        raise ValueError(f"loop body returned {len(r)} values for {n} loop variables")
    body_produced = set(sd.variables) - before
    nexts = [sd._op("next_iteration", [v], name=f"{frame}/NextIteration", frameName=frame) for v in r]
    for mnode, nx in zip(merge_nodes, nexts):
        mnode.inputs[1] = nx.name
    # loop invariants: outer arrays read inside the frame enter it as constants
    inside = cond_produced | body_produced | {m.name for m in merges} | {i.name for i in idents} | {lc.name} | \
        {s[k].name for s in switches for k in (0, 1)} | {e.name for e in enters} | {x.name for x in nexts}
    reads = _outer_reads(sd, first_cond, inside)
    mapping = {}
    tail = sd.ops[first_cond:]
    del sd.ops[first_cond:]
    for rname in reads:
        ce = sd._op("enter", [anchored(sd.variables[rname])], name=f"{frame}/Enter_const", frameName=frame, isConstant=True)
        mapping[rname] = ce.name
    sd.ops.extend(tail)
    for node in tail:
        if node.opName == "exit":
            continue
        node.inputs = [mapping.get(i, i) if i is not None else None for i in node.inputs]
    sd._exec_plan = None
    return exits
