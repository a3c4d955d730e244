"""Op object model and executioner: ``DynamicCustomOp`` (+ builder), ``OpContext``, ``UserDefinedCustomOp`` and ``OpExecutioner``
(``nd4j-api/.../linalg/api/ops/DynamicCustomOp.java``, ``OpContext.java``, ``.../ops/executioner/OpExecutioner.java``,
``DefaultOpExecutioner.java``, ``UserDefinedCustomOp.java``).

An op object carries what the reference's carries: a name, input / output arrays and positional integer, floating-point, boolean
and data-type arguments in the order the native op reads them.  Execution turns the positional arguments into the keyword form of
the registry implementation (``ops/argschema.py``) and runs it on the device the inputs live on.
"""
from __future__ import annotations

import time

import torch

from . import argschema, registry


def _t(x):
    from ..nd.ndarray import INDArray
    if x is None:
        return None
    return x.t if isinstance(x, INDArray) else (x if isinstance(x, torch.Tensor) else torch.as_tensor(x))


def _wrap(x):
    from ..nd.ndarray import INDArray
    return INDArray(x) if isinstance(x, torch.Tensor) else x


class CustomOp:
    """What every executable op object exposes."""

    def opName(self): raise NotImplementedError
    def opHash(self): return registry.op_hash(self.opName()) if hasattr(registry, "op_hash") else hash(self.opName())
    def isInplaceCall(self): return False


class DynamicCustomOp(CustomOp):
    def __init__(self, opName, inputs=(), outputs=(), iArgs=(), tArgs=(), bArgs=(), dArgs=(), inplace=False, kwargs=None):
        registry.get(opName)                         # unknown names fail here, as the reference's descriptor lookup does
        self._name = opName
        self._in, self._out = list(inputs), list(outputs)
        self._i, self._t_, self._b, self._d = list(iArgs), list(tArgs), list(bArgs), list(dArgs)
        self._inplace, self._kw = bool(inplace), dict(kwargs or {})

    # -- builder ------------------------------------------------------------------------------------------------------------
    class Builder:
        def __init__(self, opName): self.kw = dict(opName=opName, inputs=[], outputs=[], iArgs=[], tArgs=[], bArgs=[], dArgs=[], inplace=False)
        def addInputs(self, *a): self.kw["inputs"] += list(a); return self
        def addOutputs(self, *a): self.kw["outputs"] += list(a); return self
        def addIntegerArguments(self, *a): self.kw["iArgs"] += [int(v) for v in (a[0] if len(a) == 1 and isinstance(a[0], (list, tuple)) else a)]; return self
        def addFloatingPointArguments(self, *a): self.kw["tArgs"] += [float(v) for v in (a[0] if len(a) == 1 and isinstance(a[0], (list, tuple)) else a)]; return self
        def addBooleanArguments(self, *a): self.kw["bArgs"] += [bool(v) for v in a]; return self
        def addDataTypeArguments(self, *a): self.kw["dArgs"] += list(a); return self
        def callInplace(self, flag=True): self.kw["inplace"] = bool(flag); return self
        def build(self): return DynamicCustomOp(**self.kw)

    @staticmethod
    def builder(opName): return DynamicCustomOp.Builder(opName)

    # -- accessors ----------------------------------------------------------------------------------------------------------
    def opName(self): return self._name
    def isInplaceCall(self): return self._inplace
    def inputArguments(self): return [_wrap(x) for x in self._in]
    def outputArguments(self): return [_wrap(x) for x in self._out]
    def numInputArguments(self): return len(self._in)
    def numOutputArguments(self): return len(self._out)
    def iArgs(self): return list(self._i)
    def tArgs(self): return list(self._t_)
    def bArgs(self): return list(self._b)
    def dArgs(self): return list(self._d)
    def numIArguments(self): return len(self._i)
    def numTArguments(self): return len(self._t_)
    def numBArguments(self): return len(self._b)
    def getInputArgument(self, i): return _wrap(self._in[i])
    def getOutputArgument(self, i): return _wrap(self._out[i])
    def addInputArgument(self, *a): self._in += list(a); return self
    def addOutputArgument(self, *a): self._out += list(a); return self
    def addIArgument(self, *a): self._i += [int(v) for v in a]; return self
    def addTArgument(self, *a): self._t_ += [float(v) for v in a]; return self
    def addBArgument(self, *a): self._b += [bool(v) for v in a]; return self
    def addDArgument(self, *a): self._d += list(a); return self
    def setInputArgument(self, i, a):
        while len(self._in) <= i:
            self._in.append(None)
        self._in[i] = a
    def setOutputArgument(self, i, a):
        while len(self._out) <= i:
            self._out.append(None)
        self._out[i] = a
    def clearArrays(self): self._in, self._out = [], []

    def keywordArguments(self):
        kw = argschema.kwargs_for(self._name, "CUSTOM", self._i, self._t_, self._b, dtypes=[int(getattr(d, "value", d)) for d in self._d])
        kw.update(self._kw)
        return kw

    def _run(self, inputs):
        out = registry.get(self._name).fn(*[_t(x) for x in inputs], **self.keywordArguments())
        return list(out) if isinstance(out, (tuple, list)) else [out]

    def calculateOutputShape(self, ctx=None):
        """Shapes (and types) of the outputs for the current inputs, obtained by running the op's implementation."""
        ins = ctx._in if ctx is not None else self._in
        return [{"shape": tuple(o.shape), "dataType": o.dtype} for o in self._run(ins) if isinstance(o, torch.Tensor)]

    def __repr__(self):
        return f"DynamicCustomOp({self._name}, inputs={len(self._in)}, iArgs={self._i}, tArgs={self._t_}, bArgs={self._b})"


class OpContext:
    """Arrays and arguments of one execution, kept apart from the op object so that one op can be run from several threads."""

    def __init__(self):
        self._in, self._out, self._i, self._t_, self._b, self._d = [], [], [], [], [], []

    def setInputArray(self, i, arr):
        while len(self._in) <= i:
            self._in.append(None)
        self._in[i] = arr
    def setInputArrays(self, *arrs): self._in = list(arrs[0]) if len(arrs) == 1 and isinstance(arrs[0], (list, tuple)) else list(arrs)
    def setOutputArray(self, i, arr):
        while len(self._out) <= i:
            self._out.append(None)
        self._out[i] = arr
    def setOutputArrays(self, *arrs): self._out = list(arrs[0]) if len(arrs) == 1 and isinstance(arrs[0], (list, tuple)) else list(arrs)
    def setIArguments(self, *a): self._i = [int(v) for v in a]
    def setTArguments(self, *a): self._t_ = [float(v) for v in a]
    def setBArguments(self, *a): self._b = [bool(v) for v in a]
    def setDArguments(self, *a): self._d = list(a)
    def getInputArrays(self): return [_wrap(x) for x in self._in]
    def getOutputArrays(self): return [_wrap(x) for x in self._out]
    def getInputArray(self, i): return _wrap(self._in[i])
    def getOutputArray(self, i): return _wrap(self._out[i])
    def numInputArguments(self): return len(self._in)
    def numOutputArguments(self): return len(self._out)
    def getIArguments(self): return list(self._i)
    def getTArguments(self): return list(self._t_)
    def getBArguments(self): return list(self._b)
    def purge(self): self.__init__()
    def close(self): self.purge()


class UserDefinedCustomOp(CustomOp):
    """A user-defined op: subclasses give ``opName``, ``exec(inputs) -> outputs`` on tensors and optionally ``doDiff(inputs, outputs,
    gradients) -> input gradients``; without ``doDiff`` autograd differentiates through ``exec``.  ``SameDiff.doUdf`` puts an
    instance into a graph."""

    def opName(self): return type(self).__name__
    def exec(self, inputs): raise NotImplementedError
    def doDiff(self, inputs, outputs, gradients): return None
    def numOutputs(self): return 1
    def configureFromArguments(self): return None
    def configureWithSameDiff(self, sd): return None

    def register(self):
        """Makes the op executable by name (graphs that contain it can then be saved and, with the class imported, loaded)."""
        udf = self

        class _Fn(torch.autograd.Function):
            @staticmethod
            def forward(ctx, *ins):
                with torch.enable_grad():
                    outs = udf.exec(list(ins))
                outs = list(outs) if isinstance(outs, (tuple, list)) else [outs]
                ctx.save_for_backward(*ins, *outs)
                ctx.n_in = len(ins)
                return tuple(o.detach() for o in outs) if len(outs) > 1 else outs[0].detach()

            @staticmethod
            def backward(ctx, *grads):
                saved = ctx.saved_tensors
                ins, outs = list(saved[:ctx.n_in]), list(saved[ctx.n_in:])
                g = udf.doDiff(ins, outs, list(grads))
                return tuple(g)

        def fn(*ins, **kw):
            has_diff = type(udf).doDiff is not UserDefinedCustomOp.doDiff
            return _Fn.apply(*ins) if has_diff else udf.exec(list(ins))
        registry.op(self.opName(), n_out=self.numOutputs(), group="udf")(fn)
        return self


class ProfilingMode:
    DISABLED, NAN_PANIC, INF_PANIC, ANY_PANIC, OPERATIONS, ALL = "DISABLED", "NAN_PANIC", "INF_PANIC", "ANY_PANIC", "OPERATIONS", "ALL"


class OpExecutioner:
    _instance = None

    def __init__(self):
        self.verbose = self.debug = False
        self.profilingMode = ProfilingMode.DISABLED
        self.lastOp = None
        self.stats = {}                 # op name -> [invocations, seconds]

    @classmethod
    def instance(cls):
        if cls._instance is None:
            cls._instance = OpExecutioner()
        return cls._instance

    # -- configuration ------------------------------------------------------------------------------------------------------
    def enableVerboseMode(self, flag=True): self.verbose = bool(flag)
    def enableDebugMode(self, flag=True): self.debug = bool(flag)
    def isVerbose(self): return self.verbose
    def isDebug(self): return self.debug
    def setProfilingMode(self, mode): self.profilingMode = mode
    def getProfilingMode(self): return self.profilingMode
    def getLastOp(self): return self.lastOp
    def type(self): return "CUDA" if torch.cuda.is_available() else "NATIVE_CPU"

    def getEnvironmentInformation(self):
        info = {"backend": "deeplearning4j_b200", "torch": torch.__version__, "cuda.available": torch.cuda.is_available()}
        if torch.cuda.is_available():
            p = torch.cuda.get_device_properties(torch.cuda.current_device())
            info.update({"cuda.deviceName": p.name, "cuda.totalMemory": p.total_memory, "cuda.multiProcessorCount": p.multi_processor_count,
                         "cuda.deviceMajor": p.major, "cuda.deviceMinor": p.minor, "cuda.numDevices": torch.cuda.device_count()})
        return info

    def printEnvironmentInformation(self):
        for k, v in self.getEnvironmentInformation().items():
            print(f"{k}: {v}")

    def commit(self):
        """Waits for everything queued on the device (``OpExecutioner.commit``)."""
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    push = commit

    # -- execution ----------------------------------------------------------------------------------------------------------
    def _check(self, name, outs):
        m = self.profilingMode
        if m in (ProfilingMode.NAN_PANIC, ProfilingMode.ANY_PANIC):
            for o in outs:
                if isinstance(o, torch.Tensor) and o.is_floating_point() and bool(torch.isnan(o).any()):
                    raise FloatingPointError(f"op '{name}' produced NaN")
        if m in (ProfilingMode.INF_PANIC, ProfilingMode.ANY_PANIC):
            for o in outs:
                if isinstance(o, torch.Tensor) and o.is_floating_point() and bool(torch.isinf(o).any()):
                    raise FloatingPointError(f"op '{name}' produced Inf")

    def exec(self, op, *inputs, context=None, **kw):
        """``exec(op)`` / ``exec(op, context)`` for op objects (returns the output arrays; preallocated outputs are filled), or
        ``exec("name", *inputs, **kwargs)`` for a registry op by name."""
        t0 = time.perf_counter() if self.profilingMode in (ProfilingMode.OPERATIONS, ProfilingMode.ALL) else None
        if isinstance(op, str):
            name = op
            out = registry.get(op).fn(*[_t(x) for x in inputs], **kw)
            outs = list(out) if isinstance(out, (tuple, list)) else [out]
            pre = []
        elif isinstance(op, UserDefinedCustomOp):
            name = op.opName()
            ins = context._in if context is not None else inputs
            out = op.exec([_t(x) for x in ins])
            outs = list(out) if isinstance(out, (tuple, list)) else [out]
            pre = context._out if context is not None else []
        else:
            name = op.opName()
            if context is None and inputs and isinstance(inputs[0], OpContext):
                context = inputs[0]
            src = context if context is not None else op
            if context is not None and (context._i or context._t_ or context._b):
                run = DynamicCustomOp(name, context._in, context._out, context._i, context._t_, context._b, context._d, kwargs=op._kw)
            else:
                run = op
            outs = run._run(src._in)
            pre = src._out
        for k, p in enumerate(pre):                 # preallocated outputs receive the result (shape-checked by copy_)
            if p is not None and k < len(outs) and isinstance(outs[k], torch.Tensor):
                _t(p).copy_(outs[k])
                outs[k] = _t(p)
        if not isinstance(op, str) and getattr(op, "isInplaceCall", lambda: False)() and outs and op._in:
            _t(op._in[0]).copy_(outs[0])
            outs[0] = _t(op._in[0])
        if not isinstance(op, str) and not pre:
            target = context if context is not None else op
            target._out = list(outs)
        self._check(name, outs)
        self.lastOp = name
        if self.verbose:
            print(f"[exec] {name}: " + ", ".join(str(tuple(o.shape)) for o in outs if isinstance(o, torch.Tensor)))
        if t0 is not None:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            s = self.stats.setdefault(name, [0, 0.0])
            s[0] += 1
            s[1] += time.perf_counter() - t0
        res = [_wrap(o) for o in outs]
        return res if not isinstance(op, str) or len(res) > 1 else res[0]

    def execAndReturn(self, op, *a, **kw):
        self.exec(op, *a, **kw)
        return op

    def calculateOutputShape(self, op, ctx=None): return op.calculateOutputShape(ctx)
    def buildContext(self): return OpContext()
    def printProfilingStats(self):
        for k, (n, s) in sorted(self.stats.items(), key=lambda kv: -kv[1][1]):
            print(f"{k:32s} {n:8d} calls {s * 1e3:10.3f} ms")
