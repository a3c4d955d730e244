"""SameDiff: define-then-run graphs with automatic differentiation.

Parity: ``nd4j-api/.../autodiff/samediff/SameDiff.java`` (graph definition ``:1606,3305-3320``,
``output`` / ``calculateGradients`` ``:1798-1929,5010``, ``fit`` ``:1929-2212``, serde
``:6218-6760``), ``SDVariable.java``, ``VariableType``.

A graph is a list of ``SameDiffOp`` nodes over named variables.  Execution walks the nodes in
definition order (which is a topological order by construction) and dispatches each node to the
op registry, so every node runs on torch / the native sm_100a kernels.  Gradients come from
torch autograd over that execution instead of a second "grad function" graph; trainable
variables live in one flat fp32 buffer (+ bf16 shadow on a B200) shared with the fused updater,
exactly like the DL4J networks.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field

import numpy as np
import torch

from ..nd.dtype import DataType
from ..nd.ndarray import INDArray, _unwrap
from ..ops import registry


class VariableType:
    VARIABLE = "VARIABLE"
    CONSTANT = "CONSTANT"
    ARRAY = "ARRAY"
    PLACEHOLDER = "PLACEHOLDER"
    SEQUENCE = "SEQUENCE"


def _tensor(x, dtype=None, device=None):
    t = _unwrap(x)
    if not isinstance(t, torch.Tensor):
        t = torch.as_tensor(np.asarray(t))
        if t.dtype == torch.float64 and dtype is None:
            t = t.float()
    if dtype is not None:
        t = t.to(dtype.to_torch() if isinstance(dtype, DataType) else dtype)
    if device is not None:
        t = t.to(device)
    return t


@dataclass
class SameDiffOp:
    name: str                 # unique node name
    opName: str               # registry name
    inputs: list              # variable names
    outputs: list             # variable names
    args: dict = field(default_factory=dict)
    controlDeps: list = field(default_factory=list)


class SDVariable:
    def __init__(self, sd, name, vtype, dtype=None, shape=None):
        self.sd, self.name, self.variableType, self._dtype, self._shape = sd, name, vtype, dtype, shape

    # ---- meta
    def getVarName(self): return self.name
    def name_(self): return self.name
    def dataType(self): return self._dtype
    def getShape(self): return self._shape
    def getVariableType(self): return self.variableType
    def isPlaceHolder(self): return self.variableType == VariableType.PLACEHOLDER
    def isConstant(self): return self.variableType == VariableType.CONSTANT

    def rename(self, new):
        self.sd.renameVariable(self.name, new)
        return self

    def getArr(self):
        return self.sd.getArrForVarName(self.name)

    def setArray(self, arr):
        self.sd.setArrayForVariable(self.name, arr)

    def eval(self, placeholders=None):
        return self.sd.output(placeholders or {}, self.name)[self.name]

    def gradient(self):
        return self.sd.grad(self.name)

    getGradient = gradient

    def markAsLoss(self):
        self.sd.addLossVariable(self.name)
        return self

    def convertToConstant(self):
        return self.sd.convertToConstant(self)

    def convertToVariable(self):
        return self.sd.convertToVariable(self)

    # ---- op sugar
    def _b(self, opn, other, rev=False):
        o = other if isinstance(other, SDVariable) else self.sd.constant(None, _scalar_like(other))
        return self.sd._op(opn, [o, self] if rev else [self, o])

    def add(self, o, *a): return self._named(o, a, "add")
    def sub(self, o, *a): return self._named(o, a, "subtract")
    def mul(self, o, *a): return self._named(o, a, "multiply")
    def div(self, o, *a): return self._named(o, a, "divide")
    def rsub(self, o, *a): return self._named(o, a, "reversesubtract")
    def rdiv(self, o, *a): return self._named(o, a, "reversedivide")
    def pow(self, p): return self.sd._op("pow", [self], p=float(p)) if not isinstance(p, SDVariable) else self._b("Pow", p)
    def mmul(self, o, *a): return self._named(o, a, "matmul")
    def dot(self, o, *dims): return self.sd._op("dot", [self, o], dimensions=list(dims))
    def neg(self): return self.sd._op("neg", [self])
    def gt(self, o): return self._b("greater", o)
    def gte(self, o): return self._b("greater_equal", o)
    def lt(self, o): return self._b("less", o)
    def lte(self, o): return self._b("less_equal", o)
    def eq(self, o): return self._b("equals", o)
    def neq(self, o): return self._b("not_equals", o)
    def squaredDifference(self, o): return self._b("squaredsubtract", o)

    def _named(self, o, a, opn):
        # DL4J allows x.add("name", y)
        if isinstance(o, str) and a:
            return self.sd._op(opn, [self, a[0] if isinstance(a[0], SDVariable) else self.sd.constant(None, _scalar_like(a[0]))], name=o)
        return self._b(opn, o)

    __add__ = lambda s, o: s._b("add", o)
    __radd__ = lambda s, o: s._b("add", o, True)
    __sub__ = lambda s, o: s._b("subtract", o)
    __rsub__ = lambda s, o: s._b("subtract", o, True)
    __mul__ = lambda s, o: s._b("multiply", o)
    __rmul__ = lambda s, o: s._b("multiply", o, True)
    __truediv__ = lambda s, o: s._b("divide", o)
    __rtruediv__ = lambda s, o: s._b("divide", o, True)
    __neg__ = neg
    __matmul__ = lambda s, o: s._b("matmul", o)

    def _r(self, opn, dims, keepDims=False, **kw):
        if dims and isinstance(dims[0], bool):
            keepDims, dims = dims[0], dims[1:]
        return self.sd._op(opn, [self], dimensions=list(dims), keepDims=keepDims, **kw)

    def sum(self, *d, keepDims=False): return self._r("reduce_sum", d, keepDims)
    def mean(self, *d, keepDims=False): return self._r("reduce_mean", d, keepDims)
    def prod(self, *d, keepDims=False): return self._r("reduce_prod", d, keepDims)
    def max(self, *d, keepDims=False): return self._r("reduce_max", d, keepDims)
    def min(self, *d, keepDims=False): return self._r("reduce_min", d, keepDims)
    def norm1(self, *d, keepDims=False): return self._r("reduce_norm1", d, keepDims)
    def norm2(self, *d, keepDims=False): return self._r("reduce_norm2", d, keepDims)
    def normmax(self, *d, keepDims=False): return self._r("reduce_norm_max", d, keepDims)
    def std(self, biasCorrected=True, *d, keepDims=False): return self._r("reduce_stdev", d, keepDims, biasCorrected=biasCorrected)
    def var(self, biasCorrected=True, *d, keepDims=False): return self._r("reduce_variance", d, keepDims, biasCorrected=biasCorrected)
    def argmax(self, *d, keepDims=False): return self._r("argmax", d, keepDims)
    def argmin(self, *d, keepDims=False): return self._r("argmin", d, keepDims)

    def reshape(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (list, tuple)):
            shape = shape[0]
        if len(shape) == 1 and isinstance(shape[0], SDVariable):
            return self.sd._op("reshape", [self, shape[0]])
        return self.sd._op("reshape", [self], shape=[int(s) for s in shape])

    def permute(self, *dims):
        if len(dims) == 1 and isinstance(dims[0], (list, tuple)):
            dims = dims[0]
        return self.sd._op("permute", [self], dimensions=[int(d) for d in dims])

    def transpose(self): return self.sd._op("transpose", [self])
    def castTo(self, dtype): return self.sd._op("cast", [self], dtype=int(dtype))

    def get(self, *idx):
        return self.sd._op("strided_slice", [self], **_sd_index(idx))

    def __getitem__(self, item):
        return self.sd._op("__getitem__", [self], index=item if isinstance(item, tuple) else (item,))

    def shape(self): return self.sd._op("shape_of", [self])
    def rank(self): return self.sd._op("rank", [self])
    def length(self): return self.sd._op("size", [self])

    def __repr__(self):
        return f"SDVariable(name=\"{self.name}\", variableType={self.variableType}, dtype={getattr(self._dtype, 'name', self._dtype)}, shape={self._shape})"


def _scalar_like(v):
    if isinstance(v, bool):
        return torch.tensor(v)
    if isinstance(v, int):
        return torch.tensor(float(v))
    if isinstance(v, float):
        return torch.tensor(v, dtype=torch.float32)
    return _tensor(v)


def _sd_index(idx):
    from ..nd.ndarray import NDArrayIndex
    begin, end, strides, bm, em, sm = [], [], [], 0, 0, 0
    for i, ix in enumerate(idx):
        if isinstance(ix, NDArrayIndex):
            if ix.kind == "all":
                begin.append(0); end.append(0); strides.append(1); bm |= 1 << i; em |= 1 << i
            elif ix.kind == "point":
                begin.append(ix.a); end.append(ix.a + 1); strides.append(1); sm |= 1 << i
            else:
                begin.append(ix.a); end.append(ix.b); strides.append(ix.step)
        else:
            begin.append(int(ix)); end.append(int(ix) + 1); strides.append(1); sm |= 1 << i
    return dict(begin=begin, end=end, strides=strides, begin_mask=bm, end_mask=em, shrink_axis_mask=sm)


registry.op("__getitem__")(lambda x, index=(), **kw: x[index])


class NameScope:
    def __init__(self, sd, name):
        self.sd, self.name = sd, name

    def __enter__(self):
        self.sd._scopes.append(self.name)
        return self

    def __exit__(self, *a):
        self.sd._scopes.pop()

    close = __exit__


class SameDiff:
    def __init__(self):
        self.variables: dict[str, SDVariable] = {}
        self.arrays: dict[str, torch.Tensor] = {}       # VARIABLE / CONSTANT values (and bound placeholders)
        self.ops: list[SameDiffOp] = []
        self._producer: dict[str, SameDiffOp] = {}
        self.lossVariables: list[str] = []
        self.trainingConfig = None
        self.listeners = []
        self._scopes: list[str] = []
        self._counter = itertools.count()
        self._grads: dict[str, torch.Tensor] = {}
        self.device = torch.device("cpu")
        self._training = None          # TrainingSession state (flat buffers, updater)
        self._weight_inits = {}
        self.metadata = {}
        self._exec_plan = None

    @staticmethod
    def create():
        return SameDiff()

    # ------------------------------------------------------------------ namespaces
    @property
    def math(self):
        from .namespaces import SDMath
        return SDMath(self)

    @property
    def nn(self):
        from .namespaces import SDNN
        return SDNN(self)

    @property
    def cnn(self):
        from .namespaces import SDCNN
        return SDCNN(self)

    @property
    def rnn(self):
        from .namespaces import SDRNN
        return SDRNN(self)

    @property
    def loss(self):
        from .namespaces import SDLoss
        return SDLoss(self)

    @property
    def linalg(self):
        from .namespaces import SDLinalg
        return SDLinalg(self)

    @property
    def image(self):
        from .namespaces import SDImage
        return SDImage(self)

    @property
    def bitwise(self):
        from .namespaces import SDBitwise
        return SDBitwise(self)

    @property
    def random(self):
        from .namespaces import SDRandom
        return SDRandom(self)

    def __getattr__(self, item):
        # SDBaseOps methods are available directly on the SameDiff instance
        if item.startswith("_"):
            raise AttributeError(item)
        from .namespaces import SDBaseOps
        base = SDBaseOps(self)
        if hasattr(base, item):
            return getattr(base, item)
        raise AttributeError(item)

    # ------------------------------------------------------------------ naming
    def withNameScope(self, name):
        return NameScope(self, name)

    def currentNameScope(self):
        return "/".join(self._scopes) if self._scopes else None

    def _unique(self, base):
        if self._scopes:
            base = "/".join(self._scopes) + "/" + base
        if base not in self.variables and base not in {o.name for o in self.ops[-1:]}:
            if base not in self.variables:
                return base
        i = 1
        while f"{base}_{i}" in self.variables:
            i += 1
        return f"{base}_{i}"

    # ------------------------------------------------------------------ variable creation
    def _add_var(self, name, vtype, dtype, shape):
        if name in self.variables:
            raise ValueError(f"variable '{name}' already exists")
        v = SDVariable(self, name, vtype, dtype, tuple(shape) if shape is not None else None)
        self.variables[name] = v
        self._exec_plan = None
        return v

    def placeHolder(self, name, dtype=DataType.FLOAT, *shape):
        if len(shape) == 1 and isinstance(shape[0], (list, tuple)):
            shape = shape[0]
        return self._add_var(self._scoped(name), VariableType.PLACEHOLDER, dtype, shape)

    def _scoped(self, name):
        """Explicit names are prefixed with the active name scope (``SameDiff.java`` ``withNameScope``)."""
        return "/".join(self._scopes) + "/" + name if self._scopes else name

    def var(self, name=None, *args, dtype=None, shape=None, weightInit=None):
        """``var(name, array)``, ``var(name, dtype, *shape)``, ``var(name, weightInitScheme, dtype, *shape)``."""
        from ..nn.weights import IWeightInit, WeightInit
        arr, wi = None, weightInit
        rest = list(args)
        if rest and isinstance(rest[0], (torch.Tensor, INDArray, np.ndarray)):
            arr = _tensor(rest.pop(0))
        if rest and (isinstance(rest[0], IWeightInit) or (isinstance(rest[0], str) and rest[0].upper() in WeightInit._MAP)):
            wi = WeightInit.get(rest.pop(0))
        if rest and isinstance(rest[0], DataType):
            dtype = rest.pop(0)
        if rest:
            shape = rest[0] if len(rest) == 1 and isinstance(rest[0], (list, tuple)) else rest
        name = self._scoped(name) if name else self._unique("sd_var")
        if arr is None:
            dtype = dtype or DataType.FLOAT
            shape = tuple(int(s) for s in shape)
            arr = torch.zeros(shape, dtype=dtype.to_torch())
            wi = WeightInit.get(wi) if wi is not None else None
            if wi is not None:
                fan_in = shape[0] if len(shape) >= 1 else 1
                fan_out = shape[1] if len(shape) >= 2 else fan_in
                if len(shape) > 2:
                    rf = int(np.prod(shape[2:]))
                    fan_in, fan_out = shape[1] * rf, shape[0] * rf
                import zlib
                g = torch.Generator().manual_seed(zlib.crc32(name.encode()) & 0x7FFFFFFF)   # same on every rank and run
                tmp = torch.empty(shape, dtype=torch.float32)
                wi.init(fan_in, fan_out, tmp, g)
                arr = tmp.to(dtype.to_torch())
                self._weight_inits[name] = wi
        v = self._add_var(name, VariableType.VARIABLE, DataType.from_torch(arr.dtype), arr.shape)
        self.arrays[name] = arr.to(self.device)
        self._training = None
        return v

    def constant(self, name=None, value=None):
        if value is None and not isinstance(name, str):
            name, value = None, name
        t = _scalar_like(value) if not isinstance(value, (torch.Tensor, INDArray, np.ndarray)) else _tensor(value)
        name = self._scoped(name) if name else self._unique("const")
        v = self._add_var(name, VariableType.CONSTANT, DataType.from_torch(t.dtype), t.shape)
        self.arrays[name] = t.to(self.device)
        return v

    def zero(self, name, dtype=DataType.FLOAT, *shape):
        return self.var(name, torch.zeros([int(s) for s in shape], dtype=dtype.to_torch()))

    def one(self, name, dtype=DataType.FLOAT, *shape):
        return self.var(name, torch.ones([int(s) for s in shape], dtype=dtype.to_torch()))

    def scalar(self, name, value, dtype=None):
        return self.constant(name, torch.tensor(value, dtype=(dtype or DataType.FLOAT).to_torch()))

    # ------------------------------------------------------------------ lookups
    def getVariable(self, name): return self.variables[name]
    def hasVariable(self, name): return name in self.variables
    def variableMap(self): return dict(self.variables)
    def getVariables(self): return list(self.variables.values())
    variablesList = getVariables
    def inputs(self): return [n for n, v in self.variables.items() if v.variableType == VariableType.PLACEHOLDER]
    def getOps(self): return list(self.ops)
    def getOpById(self, name): return next(o for o in self.ops if o.name == name)

    def outputs(self):
        consumed = {i for o in self.ops for i in o.inputs}
        return [n for o in self.ops for n in o.outputs if n not in consumed]

    def trainableVariables(self):
        return [v for v in self.variables.values() if v.variableType == VariableType.VARIABLE
                and v._dtype is not None and v._dtype.is_fp()]

    def getArrForVarName(self, name):
        t = self.arrays.get(name)
        if t is None:
            t = self.__dict__.get("_eager_arrays", {}).get(name)
        return None if t is None else INDArray(t)

    def setArrayForVariable(self, name, arr):
        t = _tensor(arr).to(self.device)
        cur = self.arrays.get(name)
        if cur is not None and cur.shape == t.shape and self._training is not None and name in self._training.views:
            with torch.no_grad():
                cur.copy_(t.to(cur.dtype))
            self._training.refresh_shadow()
        else:
            self.arrays[name] = t
        v = self.variables[name]
        v._shape, v._dtype = tuple(t.shape), DataType.from_torch(t.dtype)

    associateArrayWithVariable = lambda self, arr, var: self.setArrayForVariable(var.name if isinstance(var, SDVariable) else var, arr)

    def renameVariable(self, old, new):
        v = self.variables.pop(old)
        v.name = new
        self.variables[new] = v
        if old in self.arrays:
            self.arrays[new] = self.arrays.pop(old)
        for o in self.ops:
            o.inputs = [new if i == old else i for i in o.inputs]
            o.outputs = [new if i == old else i for i in o.outputs]
        if old in self._producer:
            self._producer[new] = self._producer.pop(old)
        self.lossVariables = [new if l == old else l for l in self.lossVariables]
        self._exec_plan = None

    def convertToConstant(self, v):
        v = v if isinstance(v, SDVariable) else self.variables[v]
        v.variableType = VariableType.CONSTANT
        self._training = None
        return v

    def convertToVariable(self, v):
        v = v if isinstance(v, SDVariable) else self.variables[v]
        v.variableType = VariableType.VARIABLE
        self._training = None
        return v

    convertToConstants = lambda self, vs: [self.convertToConstant(v) for v in vs]
    convertToVariables = lambda self, vs: [self.convertToVariable(v) for v in vs]

    # ------------------------------------------------------------------ op creation
    def _op(self, opName, inputs, n_out=None, name=None, **args):
        d = registry.get(opName)
        ins = []
        for i in inputs:
            if i is None:
                ins.append(None)
            elif isinstance(i, SDVariable):
                ins.append(i.name)
            else:
                ins.append(self.constant(None, i).name)
        n = n_out if n_out is not None else (d.n_out if d.n_out > 0 else 1)
        base = name or opName
        node_name = self._unique(base)
        outs = []
        for k in range(n):
            on = node_name if k == 0 else f"{node_name}:{k}"
            if name and k == 0:
                on = node_name
            outs.append(self._add_var(on, VariableType.ARRAY, None, None))
        node = SameDiffOp(node_name, opName, ins, [o.name for o in outs], {k: v for k, v in args.items() if v is not None})
        self.ops.append(node)
        for o in outs:
            self._producer[o.name] = node
        self._exec_plan = None
        if getattr(self, "_eager", False):
            self._eager_run(node, d)
        return outs[0] if n == 1 else outs

    # ------------------------------------------------------------------ eager mode (SameDiff.enableEagerMode)
    def enableEagerMode(self):
        """Every op added from now on is also executed at once when the arrays of all its inputs are known (variables, constants,
        placeholders that were given an array with ``setArray``, results of earlier eager ops); ``SDVariable.getArr`` then returns
        the value while the graph is still being defined."""
        self._eager = True
        self.__dict__.setdefault("_eager_arrays", {})
        return self

    def isEagerMode(self):
        return bool(getattr(self, "_eager", False))

    def _eager_run(self, node, d):
        vals = []
        for i in node.inputs:
            if i is None:
                vals.append(None)
                continue
            t = self.arrays.get(i)
            if t is None:
                t = self._eager_arrays.get(i)
            if t is None:
                return                                  # an input without a value yet (a placeholder): the op stays symbolic
            vals.append(t)
        with torch.no_grad():
            out = d.fn(*vals, **node.args)
        outs = list(out) if isinstance(out, (tuple, list)) else [out]
        for name, t in zip(node.outputs, outs):
            if isinstance(t, torch.Tensor):
                self._eager_arrays[name] = t

    def doUdf(self, udf, *inputs, name=None):
        """Adds a user-defined op (``ops.executioner.UserDefinedCustomOp``) to the graph (``SameDiff.doUdf``)."""
        udf.register()
        udf.configureWithSameDiff(self)
        return self._op(udf.opName(), list(inputs), n_out=udf.numOutputs(), name=name)

    @staticmethod
    def collectTrace(traces=None):
        """Rebuild a graph from eagerly executed ops (``SameDiff.collectTrace``): arrays produced by one traced op and consumed by a
        later one become edges, every other input becomes a constant holding the value it had."""
        from ..ops import registry as reg
        traces = list(reg.TRACES) if traces is None else list(traces)
        sd = SameDiff.create()
        known = {}                                   # id(tensor) -> SDVariable
        keep = []                                    # keeps traced tensors alive so ids stay unique
        for tr in traces:
            ins = []
            for t in tr.inputs:
                if t is None:
                    ins.append(None)
                    continue
                v = known.get(id(t))
                if v is None:
                    v = sd.constant(None, t.detach() if isinstance(t, torch.Tensor) else t)
                    known[id(t)] = v
                    keep.append(t)
                ins.append(v)
            outs = sd._op(tr.opName, ins, n_out=len(tr.outputs), **tr.args)
            outs = outs if isinstance(outs, list) else [outs]
            for o, t in zip(outs, tr.outputs):
                known[id(t)] = o
                keep.append(t)
        return sd

    def invokeGraphOn(self, other):
        for n, v in self.variables.items():
            if n not in other.variables:
                other.variables[n] = SDVariable(other, n, v.variableType, v._dtype, v._shape)
                if n in self.arrays:
                    other.arrays[n] = self.arrays[n]
        for o in self.ops:
            node = SameDiffOp(o.name, o.opName, list(o.inputs), list(o.outputs), dict(o.args))
            other.ops.append(node)
            for out in node.outputs:
                other._producer[out] = node
        return other.variables[self.outputs()[-1]] if self.ops else None

    # ------------------------------------------------------------------ control flow
    def ifCond(self, *a):
        """``ifCond([outputName, ifName,] cond_fn, true_fn, false_fn)`` (``ControlFlow.java:139``): the lambdas build sub-graphs over
        this instance; the result is a ``merge`` of the two branches, each gated by ``switch`` nodes on the predicate, so only the
        taken branch executes and the construct is part of the serialised graph."""
        from .controlflow import build_if
        fns = [f for f in a if callable(f)]
        names = [n for n in a if isinstance(n, str) or n is None]
        cond, tb, fb = fns
        return build_if(self, cond, tb, fb, name=names[0] if names and names[0] else None)

    def whileLoop(self, *a):
        """``whileLoop([outputNames, loopName,] loopVars, cond, body)`` (``SameDiff.java`` ``whileLoop``).

        ``cond`` / ``body`` are either SameDiff lambdas ``(sd, SDVariable[]) -> SDVariable | SDVariable[]`` that define ops on
        this instance -- the loop then becomes an ``enter / merge / loop_cond / switch / exit / next_iteration`` frame in the
        graph (``ControlFlow.java:505``), which serialises and runs on the frame-aware executor -- or plain callables over
        torch tensors ``(*tensors) -> tensor(s)``, which run eagerly inside one opaque ``while_loop`` node."""
        import inspect
        loop_vars = list(next(x for x in a if isinstance(x, (list, tuple)) and x and isinstance(x[0], SDVariable)))
        fns = [f for f in a if callable(f)]
        cond_fn, body_fn = fns
        try:
            graph_mode = len(inspect.signature(cond_fn).parameters) == 2
        except (TypeError, ValueError):
            graph_mode = False
        if not graph_mode:
            sub = (self, cond_fn, body_fn, len(loop_vars))
            outs = self._op("while_loop", loop_vars, n_out=len(loop_vars), body=sub)
            return outs if isinstance(outs, list) else [outs]
        from .controlflow import build_while
        loop_name = next((x for x in a if isinstance(x, str)), None)
        return build_while(self, loop_vars, cond_fn, body_fn, name=loop_name)

    # ------------------------------------------------------------------ loss / training config
    def setLossVariables(self, *names):
        if len(names) == 1 and isinstance(names[0], (list, tuple)):
            names = names[0]
        self.lossVariables = [n.name if isinstance(n, SDVariable) else n for n in names]

    def addLossVariable(self, n):
        n = n.name if isinstance(n, SDVariable) else n
        if n not in self.lossVariables:
            self.lossVariables.append(n)

    def getLossVariables(self): return list(self.lossVariables)

    def setTrainingConfig(self, tc):
        self.trainingConfig = tc
        self._training = None

    def getTrainingConfig(self): return self.trainingConfig
    def setListeners(self, *ls): self.listeners = list(ls[0]) if len(ls) == 1 and isinstance(ls[0], (list, tuple)) else list(ls)
    def addListeners(self, *ls): self.listeners.extend(ls)
    def getListeners(self): return self.listeners

    # ------------------------------------------------------------------ execution
    def to(self, device):
        self.device = torch.device(device)
        self.arrays = {k: v.to(self.device) for k, v in self.arrays.items()}
        self._training = None
        return self

    def _needed_ops(self, outputs):
        need, stack = set(), list(outputs)
        order = []
        seen_nodes = set()
        while stack:
            n = stack.pop()
            if n in need:
                continue
            need.add(n)
            p = self._producer.get(n)
            if p is not None and id(p) not in seen_nodes:
                seen_nodes.add(id(p))
                stack.extend(i for i in p.inputs if i is not None)
        return [o for o in self.ops if id(o) in seen_nodes]

    def _exec(self, placeholders, outputs, values=None, training=False, listeners_at=None):
        """Run the sub-graph needed for ``outputs``; returns the full value table."""
        from .session import InferenceSession
        return InferenceSession(self).run(placeholders, outputs, values, training)

    def output(self, placeholders=None, *outputs):
        if outputs and isinstance(outputs[0], (list, tuple)):
            outputs = tuple(outputs[0])
        if hasattr(placeholders, "getFeatures"):
            placeholders = self._ds_to_placeholders(placeholders)
        outs = [o.name if isinstance(o, SDVariable) else o for o in outputs] or self.outputs()
        with torch.no_grad():
            vals = self._exec(placeholders or {}, outs)
        return {o: INDArray(vals[o]) if isinstance(vals[o], torch.Tensor) else vals[o] for o in outs}

    exec = output
    batchOutput = lambda self: _BatchOutput(self)

    def outputSingle(self, placeholders, output):
        return list(self.output(placeholders, output).values())[0]

    def outputAll(self, placeholders):
        return self.output(placeholders, *[n for n, v in self.variables.items() if v.variableType == VariableType.ARRAY])

    def calculateGradients(self, placeholders, *wrt):
        if wrt and isinstance(wrt[0], (list, tuple)):
            wrt = tuple(wrt[0])
        wrt = [w.name if isinstance(w, SDVariable) else w for w in wrt] or [v.name for v in self.trainableVariables()]
        if not self.lossVariables:
            raise ValueError("no loss variables set: call setLossVariables(...) first")
        from .session import InferenceSession
        leaves = {}
        for w in wrt:
            base = self.arrays[w] if w in self.arrays else _tensor(placeholders[w]).to(self.device)
            leaves[w] = base.detach().clone().requires_grad_(True)
        with torch.enable_grad():
            vals = InferenceSession(self).run(placeholders or {}, self.lossVariables, dict(leaves), training=True)
            loss = sum(vals[l].sum() for l in self.lossVariables)
        grads = torch.autograd.grad(loss, [leaves[w] for w in wrt], allow_unused=True)
        out = {}
        for w, g in zip(wrt, grads):
            g = g if g is not None else torch.zeros_like(leaves[w])
            self._grads[w] = g
            out[w] = INDArray(g)
        return out

    def grad(self, name):
        g = self._grads.get(name)
        return None if g is None else INDArray(g)

    def createGradFunction(self, *a):
        """Kept for API parity: differentiation happens through autograd at execution time."""
        return None

    def _ds_to_placeholders(self, ds):
        tc = self.trainingConfig
        if tc is None:
            raise ValueError("a TrainingConfig with feature/label mappings is required to feed DataSets")
        return tc.placeholders_from(ds)

    # ------------------------------------------------------------------ training
    def fit(self, data=None, epochs=1, *a, **kw):
        from .training import fit as _fit
        return _fit(self, data, epochs, *a, **kw)

    def evaluate(self, iterator, outputVariable, *evals):
        out = outputVariable.name if isinstance(outputVariable, SDVariable) else outputVariable
        if hasattr(iterator, "reset"):
            iterator.reset()
        for ds in iterator:
            ph = self._ds_to_placeholders(ds)
            ph = {k: v for k, v in ph.items() if k in self.inputs()}
            pred = self.output(ph, out)[out]
            labels = ds.getLabels() if hasattr(ds, "getLabels") and not isinstance(ds.getLabels(), list) else ds.getLabels(0)
            for e in evals:
                e.eval(labels, pred)
        return evals[0] if len(evals) == 1 else list(evals)

    # ------------------------------------------------------------------ serde
    def asFlatBuffers(self, saveUpdaterState=True):
        from .serde.flatgraph import to_flatbuffers
        return to_flatbuffers(self, saveUpdaterState)

    @staticmethod
    def fromFlatBuffers(buf, loadUpdaterState=True):
        from .serde.flatgraph import from_flatbuffers
        return from_flatbuffers(buf, loadUpdaterState)

    def asFlatFile(self, path, saveUpdaterState=True):
        with open(path, "wb") as f:
            f.write(self.asFlatBuffers(saveUpdaterState))

    @staticmethod
    def fromFlatFile(path, loadUpdaterState=True):
        with open(path, "rb") as f:
            return SameDiff.fromFlatBuffers(f.read(), loadUpdaterState)

    def save(self, path, saveUpdaterState=True):
        from .serde.sdnb import save as _save
        _save(self, path, saveUpdaterState)

    @staticmethod
    def load(path, loadUpdaterState=True):
        from .serde.sdnb import load as _load
        return _load(path, loadUpdaterState)

    def saveAsSDZ(self, path, saveUpdaterState=True):
        from .serde.sdnb import save_sdz
        save_sdz(self, path, saveUpdaterState)

    @staticmethod
    def loadSDZ(path, loadUpdaterState=True):
        from .serde.sdnb import load_sdz
        return load_sdz(path, loadUpdaterState)

    def summary(self):
        lines = ["--- Summary ---", f"Variables:               {len(self.variables)}",
                 f"Functions:               {len(self.ops)}", f"Loss variables:          {self.lossVariables}", "",
                 f"{'- Name -':<40}{'- Type -':<14}{'- Data Type -':<14}- Shape -"]
        for n, v in self.variables.items():
            lines.append(f"{n:<40}{v.variableType:<14}{getattr(v._dtype, 'name', '-'):<14}{v._shape}")
        lines += ["", "--- Functions ---", f"{'- Function Name -':<36}{'- Op -':<34}- Inputs -> Outputs -"]
        for o in self.ops:
            lines.append(f"{o.name:<36}{o.opName:<34}{o.inputs} -> {o.outputs}")
        return "\n".join(lines)

    def dup(self):
        sd = SameDiff()
        sd.device = self.device
        for n, v in self.variables.items():
            sd.variables[n] = SDVariable(sd, n, v.variableType, v._dtype, v._shape)
        sd.arrays = {k: v.clone() for k, v in self.arrays.items()}
        for o in self.ops:
            node = SameDiffOp(o.name, o.opName, list(o.inputs), list(o.outputs), dict(o.args), list(o.controlDeps))
            sd.ops.append(node)
            for out in node.outputs:
                sd._producer[out] = node
        sd.lossVariables = list(self.lossVariables)
        sd.trainingConfig = self.trainingConfig
        return sd


class _BatchOutput:
    def __init__(self, sd):
        self.sd, self.ph, self.outs = sd, {}, []

    def input(self, name, arr):
        self.ph[name.name if isinstance(name, SDVariable) else name] = arr
        return self

    def inputs(self, m):
        self.ph.update(m)
        return self

    def output(self, *names):
        self.outs.extend(n.name if isinstance(n, SDVariable) else n for n in names)
        return self

    def exec(self):
        return self.sd.output(self.ph, *self.outs)

    def outputSingle(self):
        return list(self.exec().values())[0]

    execSingle = outputSingle
