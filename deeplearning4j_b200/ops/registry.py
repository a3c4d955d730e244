"""Declarable-op registry: op name -> implementation over torch tensors.

Replaces ``OpRegistrator`` / ``DeclarableOp`` (``libnd4j/include/ops/declarable/OpRegistrator.h:64-131``,
``impl/DeclarableOp.cpp:866-1085``).  Names are the libnd4j op names (the identities stored in
``FlatNode.opName``); ``op_hash`` reproduces ``HashUtil.getLongHash`` so CUSTOM ops keep their
``opNum``.  Implementations live in ``ops/impl_*.py`` and register themselves on import.
"""
from __future__ import annotations

import importlib
from dataclasses import dataclass, field
from typing import Callable

_IMPL_MODULES = ("impl_elementwise", "impl_reduce", "impl_shape", "impl_nn", "impl_conv", "impl_loss", "impl_rnn",
                 "impl_linalg", "impl_random", "impl_image", "impl_misc", "impl_updaters", "impl_legacy")


@dataclass
class OpDef:
    name: str
    fn: Callable
    n_out: int = 1               # -1 = variable number of outputs (returns a sequence)
    group: str = ""
    differentiable: bool = True
    aliases: tuple = ()


REGISTRY: dict[str, OpDef] = {}
_loaded = False


def op(name, *aliases, n_out=1, group="", differentiable=True):
    def deco(fn):
        d = OpDef(name, fn, n_out, group or fn.__module__.rsplit("impl_", 1)[-1], differentiable, tuple(aliases))
        REGISTRY[name] = d
        for a in aliases:
            REGISTRY[a] = d
        return fn
    return deco


def load_all():
    global _loaded
    if _loaded:
        return REGISTRY
    for m in _IMPL_MODULES:
        importlib.import_module(f"deeplearning4j_b200.ops.{m}")
    _loaded = True
    return REGISTRY


def get(name: str) -> OpDef:
    load_all()
    d = REGISTRY.get(name)
    if d is None:
        raise KeyError(f"op '{name}' is not registered")
    return d


def has(name: str) -> bool:
    load_all()
    return name in REGISTRY


# ----------------------------------------------------------------------------- execution trace
# ``NativeOps.toggleOpTrace / listOpTraces / purgeOpTrace`` + ``OpExecTrace``: while tracing is on, every eagerly executed op
# is recorded with its arguments and the identity of its input / output arrays, from which ``SameDiff.collectTrace`` rebuilds a graph.
TRACE_ON = False
TRACES = []


class OpExecTrace:
    def __init__(self, opName, inputs, outputs, args):
        self.opName, self.inputs, self.outputs, self.args = opName, inputs, outputs, args

    def inputShapes(self): return [tuple(t.shape) if hasattr(t, "shape") else None for t in self.inputs]
    def outputShapes(self): return [tuple(t.shape) if hasattr(t, "shape") else None for t in self.outputs]

    def __repr__(self):
        return f"OpExecTrace({self.opName}, in={self.inputShapes()}, out={self.outputShapes()}, args={self.args})"


def toggle_trace(on: bool):
    global TRACE_ON
    TRACE_ON = bool(on)


def purge_traces():
    TRACES.clear()


def execute(name: str, inputs, **kwargs):
    res = get(name).fn(*inputs, **kwargs)
    if TRACE_ON:
        outs = list(res) if isinstance(res, (tuple, list)) else [res]
        TRACES.append(OpExecTrace(name, list(inputs), outs, dict(kwargs)))
    return res


def names():
    load_all()
    return sorted(REGISTRY)


# ----------------------------------------------------------------------------- HashUtil.getLongHash
_TABLE = None


def _byte_table():
    global _TABLE
    if _TABLE is None:
        h = 0x544B2FBACAAF1684
        t = []
        for _ in range(256):
            for _ in range(31):
                h = ((h >> 7) ^ h) & 0xFFFFFFFFFFFFFFFF
                h = ((h << 11) ^ h) & 0xFFFFFFFFFFFFFFFF
                h = ((h >> 10) ^ h) & 0xFFFFFFFFFFFFFFFF
            t.append(h)
        _TABLE = t
    return _TABLE


def op_hash(name: str) -> int:
    """``org.nd4j.linalg.util.HashUtil.getLongHash(String)`` (``HashUtil.java:27-78``; C++ twin
    ``libnd4j/include/helpers/impl/helper_hash.cpp:33-68``) as a signed 64-bit value."""
    HSTART, HMULT = 0xBB40E64DA205B064, 7664345821815920749
    t = _byte_table()
    h = HSTART
    for ch in name:
        c = ord(ch)
        h = ((h * HMULT) & 0xFFFFFFFFFFFFFFFF) ^ t[c & 0xFF]
        h = ((h * HMULT) & 0xFFFFFFFFFFFFFFFF) ^ t[(c >> 8) & 0xFF]
    return h - (1 << 64) if h >= (1 << 63) else h


_BY_HASH = None


def name_for_hash(h: int) -> str:
    """Inverse of :func:`op_hash` over the registered names (FlatNode.opNum -> op name)."""
    global _BY_HASH
    if _BY_HASH is None or len(_BY_HASH) != len(REGISTRY):
        load_all()
        _BY_HASH = {op_hash(n): n for n in REGISTRY}
    return _BY_HASH[int(h)]
