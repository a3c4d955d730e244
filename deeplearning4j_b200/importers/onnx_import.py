"""ONNX -> SameDiff import (``nd4j/samediff-import/samediff-import-onnx``: ``OnnxFrameworkImporter`` /
``ImportGraph`` with per-op mapping rules).  The ``.onnx`` file is parsed with the bundled protobuf wire reader, so
the ``onnx`` package is not required.  Initializers become SameDiff variables (constants when ``trainable=False``),
graph inputs become placeholders, and each node is mapped by an entry of ``OP_MAPPERS``; unknown ops raise with the
list of unsupported op types, as the reference's importer does."""
from __future__ import annotations

import numpy as np
import torch

from ..nd.dtype import DataType
from ..samediff.core import SameDiff
from . import protowire as pw

_ONNX_DTYPES = {1: np.float32, 2: np.uint8, 3: np.int8, 4: np.uint16, 5: np.int16, 6: np.int32, 7: np.int64, 9: np.bool_, 10: np.float16,
                11: np.float64, 12: np.uint32, 13: np.uint64}


def parse_tensor(buf):
    t = pw.decode(buf)
    dims = pw.packed_varints(t.get(1, []))
    dt = t.get(2, [1])[0]
    name = pw.string(t[8][0]) if 8 in t else ""
    npdt = _ONNX_DTYPES.get(dt)
    if dt == 16:                                                    # bfloat16 raw
        raw = np.frombuffer(bytes(t[9][0]), dtype=np.uint16).astype(np.uint32) << 16
        arr = raw.view(np.float32)
    elif 9 in t:
        arr = np.frombuffer(bytes(t[9][0]), dtype=np.dtype(npdt).newbyteorder("<"))
    elif 4 in t:
        arr = np.asarray(pw.packed_fixed(t[4], "f"), dtype=np.float32)
    elif 7 in t:
        arr = np.asarray(pw.packed_varints(t[7]), dtype=np.int64)
    elif 5 in t:
        arr = np.asarray(pw.packed_varints(t[5]), dtype=np.int32).astype(npdt)
    elif 10 in t:
        arr = np.asarray(pw.packed_fixed(t[10], "d"), dtype=np.float64)
    else:
        arr = np.zeros(int(np.prod(dims)) if dims else 0, dtype=npdt or np.float32)
    return name, torch.from_numpy(np.array(arr).reshape(dims) if dims else np.array(arr).reshape(()))


def parse_attribute(buf):
    a = pw.decode(buf)
    name = pw.string(a[1][0])
    typ = a.get(20, [0])[0]
    if typ == 1 or (typ == 0 and 2 in a):
        return name, pw.packed_fixed(a[2], "f")[0]
    if typ == 2 or (typ == 0 and 3 in a):
        return name, pw.signed(a[3][0])
    if typ == 3 or (typ == 0 and 4 in a):
        return name, pw.string(a[4][0])
    if typ == 4 or (typ == 0 and 5 in a):
        return name, parse_tensor(a[5][0])[1]
    if typ == 6 or (typ == 0 and 7 in a):
        return name, pw.packed_fixed(a.get(7, []), "f")
    if typ == 7 or (typ == 0 and 8 in a):
        return name, pw.packed_varints(a.get(8, []))
    if typ == 8:
        return name, [pw.string(s) for s in a.get(9, [])]
    return name, None


def parse_value_info(buf):
    v = pw.decode(buf)
    name = pw.string(v[1][0])
    shape, elem = None, 1
    if 2 in v:
        tp = pw.decode(v[2][0])
        if 1 in tp:
            tt = pw.decode(tp[1][0])
            elem = tt.get(1, [1])[0]
            if 2 in tt:
                shape = []
                for d in pw.decode(tt[2][0]).get(1, []):
                    dd = pw.decode(d)
                    shape.append(pw.signed(dd[1][0]) if 1 in dd else -1)
    return name, shape, elem


def parse_model(data):
    m = pw.decode(data)
    g = pw.decode(m[7][0])
    nodes = []
    for nb in g.get(1, []):
        n = pw.decode(nb)
        nodes.append({"inputs": [pw.string(s) for s in n.get(1, [])], "outputs": [pw.string(s) for s in n.get(2, [])],
                      "name": pw.string(n[3][0]) if 3 in n else "", "op": pw.string(n[4][0]),
                      "attrs": dict(parse_attribute(a) for a in n.get(5, []))})
    inits = dict(parse_tensor(t) for t in g.get(5, []))
    inputs = [parse_value_info(v) for v in g.get(11, [])]
    outputs = [parse_value_info(v)[0] for v in g.get(12, [])]
    opset = 13
    for o in m.get(8, []):
        od = pw.decode(o)
        if 1 not in od or pw.string(od[1][0]) in ("", "ai.onnx"):
            opset = od.get(2, [13])[0]
    return {"nodes": nodes, "initializers": inits, "inputs": inputs, "outputs": outputs, "opset": opset}


# ----------------------------------------------------------------------------- op mapping
def _const(ctx, name):
    """Value of an initializer / Constant output needed at import time (shapes, axes)."""
    if name in ctx["consts"]:
        return ctx["consts"][name]
    raise ValueError(f"importer needs '{name}' as a constant but it is computed at run time")


def _conv(sd, ctx, n, x):
    a = n["attrs"]
    w = x[1]
    k = a.get("kernel_shape")
    st, dl, pads, grp = a.get("strides", [1, 1]), a.get("dilations", [1, 1]), a.get("pads", [0, 0, 0, 0]), a.get("group", 1)
    auto = a.get("auto_pad", "NOTSET")
    return sd._op("onnx_conv", [x[0], w, x[2] if len(x) > 2 else None], strides=list(st), dilations=list(dl), pads=list(pads), group=int(grp), auto_pad=auto)


def _pool(kind):
    def f(sd, ctx, n, x):
        a = n["attrs"]
        return sd._op("onnx_pool", [x[0]], kind=kind, kernel=list(a["kernel_shape"]), strides=list(a.get("strides", [1] * len(a["kernel_shape"]))),
                      pads=list(a.get("pads", [0] * 2 * len(a["kernel_shape"]))), ceil_mode=int(a.get("ceil_mode", 0)),
                      count_include_pad=int(a.get("count_include_pad", 0)), auto_pad=a.get("auto_pad", "NOTSET"))
    return f


def _gemm(sd, ctx, n, x):
    a = n["attrs"]
    return sd._op("onnx_gemm", [x[0], x[1], x[2] if len(x) > 2 else None], alpha=float(a.get("alpha", 1.0)), beta=float(a.get("beta", 1.0)),
                  transA=int(a.get("transA", 0)), transB=int(a.get("transB", 0)))


def _reshape(sd, ctx, n, x):
    shape = [int(v) for v in _const(ctx, n["inputs"][1]).tolist()]
    return sd._op("onnx_reshape", [x[0]], shape=shape)


def _axes(ctx, n, idx=1):
    if "axes" in n["attrs"]:
        return [int(v) for v in n["attrs"]["axes"]]
    if len(n["inputs"]) > idx and n["inputs"][idx]:
        return [int(v) for v in _const(ctx, n["inputs"][idx]).reshape(-1).tolist()]
    return None


def _reduce(opn):
    def f(sd, ctx, n, x):
        ax = _axes(ctx, n)
        return sd._op(opn, [x[0]], dimensions=ax if ax is not None else [], keepDims=bool(n["attrs"].get("keepdims", 1)))
    return f


def _unary(opn): return lambda sd, ctx, n, x: sd._op(opn, [x[0]])
def _binary(opn): return lambda sd, ctx, n, x: sd._op(opn, [x[0], x[1]])


def _bn(sd, ctx, n, x):
    return sd._op("onnx_batchnorm", list(x[:5]), epsilon=float(n["attrs"].get("epsilon", 1e-5)))


def _constant(sd, ctx, n, x):
    v = n["attrs"].get("value")
    if v is None:
        for k in ("value_float", "value_int", "value_floats", "value_ints"):
            if k in n["attrs"]:
                v = torch.as_tensor(n["attrs"][k])
    ctx["consts"][n["outputs"][0]] = v
    return sd.constant(n["outputs"][0], v)


def _slice(sd, ctx, n, x):
    a = n["attrs"]
    if "starts" in a:
        starts, ends, axes, steps = a["starts"], a["ends"], a.get("axes"), None
    else:
        starts, ends = _const(ctx, n["inputs"][1]).tolist(), _const(ctx, n["inputs"][2]).tolist()
        axes = _const(ctx, n["inputs"][3]).tolist() if len(n["inputs"]) > 3 and n["inputs"][3] else None
        steps = _const(ctx, n["inputs"][4]).tolist() if len(n["inputs"]) > 4 and n["inputs"][4] else None
    return sd._op("onnx_slice", [x[0]], starts=[int(v) for v in starts], ends=[int(v) for v in ends],
                  axes=None if axes is None else [int(v) for v in axes], steps=None if steps is None else [int(v) for v in steps])


OP_MAPPERS = {
    "Add": _binary("add"), "Sub": _binary("subtract"), "Mul": _binary("multiply"), "Div": _binary("divide"), "Pow": _binary("Pow"),
    "Relu": _unary("relu"), "Sigmoid": _unary("sigmoid"), "Tanh": _unary("tanh"), "Exp": _unary("exp"), "Log": _unary("log"), "Sqrt": _unary("sqrt"),
    "Neg": _unary("neg"), "Abs": _unary("abs"), "Erf": _unary("erf"), "Identity": _unary("identity"), "Softplus": _unary("softplus"),
    "Floor": _unary("floor"), "Ceil": _unary("ceil"), "Reciprocal": _unary("reciprocal"),
    "MatMul": _binary("matmul"), "Gemm": _gemm, "Conv": _conv, "MaxPool": _pool("max"), "AveragePool": _pool("avg"),
    "GlobalAveragePool": lambda sd, ctx, n, x: sd._op("reduce_mean", [x[0]], dimensions=[2, 3], keepDims=True),
    "GlobalMaxPool": lambda sd, ctx, n, x: sd._op("reduce_max", [x[0]], dimensions=[2, 3], keepDims=True),
    "BatchNormalization": _bn, "Reshape": _reshape, "Constant": _constant, "Slice": _slice,
    "Flatten": lambda sd, ctx, n, x: sd._op("onnx_flatten", [x[0]], axis=int(n["attrs"].get("axis", 1))),
    "Softmax": lambda sd, ctx, n, x: sd._op("softmax", [x[0]], dimension=int(n["attrs"].get("axis", -1))),
    "LogSoftmax": lambda sd, ctx, n, x: sd._op("log_softmax", [x[0]], dimension=int(n["attrs"].get("axis", -1))),
    "Concat": lambda sd, ctx, n, x: sd._op("concat", list(x), concatDimension=int(n["attrs"]["axis"])),
    "Transpose": lambda sd, ctx, n, x: sd._op("permute", [x[0]], dimensions=[int(v) for v in n["attrs"]["perm"]]) if "perm" in n["attrs"] else sd._op("transpose", [x[0]]),
    "Dropout": lambda sd, ctx, n, x: sd._op("identity", [x[0]]),
    "LeakyRelu": lambda sd, ctx, n, x: sd._op("leakyrelu", [x[0]], alpha=float(n["attrs"].get("alpha", 0.01))),
    "Elu": lambda sd, ctx, n, x: sd._op("elu", [x[0]], alpha=float(n["attrs"].get("alpha", 1.0))),
    "Clip": lambda sd, ctx, n, x: sd._op("clipbyvalue", [x[0]], clipValueMin=float(n["attrs"].get("min", _const(ctx, n["inputs"][1]) if len(n["inputs"]) > 1 and n["inputs"][1] else -3.4e38)),
                                         clipValueMax=float(n["attrs"].get("max", _const(ctx, n["inputs"][2]) if len(n["inputs"]) > 2 and n["inputs"][2] else 3.4e38))),
    "ReduceMean": _reduce("reduce_mean"), "ReduceSum": _reduce("reduce_sum"), "ReduceMax": _reduce("reduce_max"), "ReduceMin": _reduce("reduce_min"),
    "Squeeze": lambda sd, ctx, n, x: sd._op("squeeze", [x[0]], dimensions=_axes(ctx, n)),
    "Unsqueeze": lambda sd, ctx, n, x: sd._op("onnx_unsqueeze", [x[0]], axes=_axes(ctx, n)),
    "Gather": lambda sd, ctx, n, x: sd._op("gather", [x[0], x[1]], axis=int(n["attrs"].get("axis", 0))),
    "Cast": lambda sd, ctx, n, x: sd._op("cast", [x[0]], dtype=int({1: DataType.FLOAT, 6: DataType.INT, 7: DataType.LONG, 9: DataType.BOOL, 10: DataType.HALF,
                                                                      11: DataType.DOUBLE, 16: DataType.BFLOAT16}[n["attrs"]["to"]])),
    "LayerNormalization": lambda sd, ctx, n, x: sd._op("layer_norm", [x[0], x[1], x[2] if len(x) > 2 else None], channelsFirst=False,
                                                       dimensions=[int(n["attrs"].get("axis", -1))]),
    "Gelu": lambda sd, ctx, n, x: sd._op("precise_gelu" if n["attrs"].get("approximate", "none") == "tanh" else "gelu_erf", [x[0]]),
    "Shape": lambda sd, ctx, n, x: sd._op("shape_of", [x[0]]),
}


# helper ops with ONNX semantics (NCHW, explicit begin/end pads) registered in the op registry
def _register_helpers():
    import torch.nn.functional as F
    from ..ops.registry import has, op
    if has("onnx_conv"):
        return

    def _pad_nd(x, pads, nd, value=0.0):
        # ONNX pads: [b1, b2, ..., e1, e2, ...] over spatial dims -> F.pad wants last dim first
        p = []
        for d in reversed(range(nd)):
            p += [pads[d], pads[d + nd]]
        return F.pad(x, p, value=value) if any(p) else x

    def _auto(x, k, s, d, auto, nd):
        pads = [0] * (2 * nd)
        for i in range(nd):
            size = x.shape[2 + i]
            out = -(-size // s[i])
            tot = max((out - 1) * s[i] + (k[i] - 1) * d[i] + 1 - size, 0)
            lo = tot // 2 if auto == "SAME_UPPER" else tot - tot // 2
            pads[i], pads[i + nd] = lo, tot - lo
        return pads

    @op("onnx_conv")
    def onnx_conv(x, w, b=None, strides=(1, 1), dilations=(1, 1), pads=(0, 0, 0, 0), group=1, auto_pad="NOTSET", **kw):
        nd = w.dim() - 2
        if auto_pad in ("SAME_UPPER", "SAME_LOWER"):
            pads = _auto(x, w.shape[2:], strides, dilations, auto_pad, nd)
        x = _pad_nd(x, list(pads), nd)
        fn = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[nd]
        return fn(x, w.to(x.dtype), None if b is None else b.to(x.dtype), tuple(strides), 0, tuple(dilations), group)

    @op("onnx_pool")
    def onnx_pool(x, kind="max", kernel=(2, 2), strides=(1, 1), pads=(0, 0, 0, 0), ceil_mode=0, count_include_pad=0, auto_pad="NOTSET", **kw):
        nd = len(kernel)
        if auto_pad in ("SAME_UPPER", "SAME_LOWER"):
            pads = _auto(x, kernel, strides, [1] * nd, auto_pad, nd)
        sym = all(pads[i] == pads[i + nd] for i in range(nd))
        if kind == "max":
            x = _pad_nd(x, list(pads), nd, float("-inf"))
            return {1: F.max_pool1d, 2: F.max_pool2d, 3: F.max_pool3d}[nd](x, tuple(kernel), tuple(strides), 0, 1, bool(ceil_mode))
        if sym:
            return {1: F.avg_pool1d, 2: F.avg_pool2d, 3: F.avg_pool3d}[nd](x, tuple(kernel), tuple(strides), tuple(pads[:nd]), bool(ceil_mode), bool(count_include_pad))
        ones = _pad_nd(torch.ones_like(x), list(pads), nd)
        xs = _pad_nd(x, list(pads), nd)
        fn = {1: F.avg_pool1d, 2: F.avg_pool2d, 3: F.avg_pool3d}[nd]
        s = fn(xs, tuple(kernel), tuple(strides), 0, bool(ceil_mode))
        return s if count_include_pad else s / fn(ones, tuple(kernel), tuple(strides), 0, bool(ceil_mode)).clamp(min=1e-12)

    @op("onnx_gemm")
    def onnx_gemm(a, b, c=None, alpha=1.0, beta=1.0, transA=0, transB=0, **kw):
        from ..ops import nnops
        a = a.t() if transA else a
        if alpha == 1.0 and beta == 1.0 and a.dim() == 2:
            return nnops.linear(a, b.t() if transB else b, c if (c is None or c.dim() <= 1) else None) + (0 if (c is None or c.dim() <= 1) else c)
        y = alpha * (a @ (b.t() if transB else b))
        return y if c is None else y + beta * c

    @op("onnx_reshape")
    def onnx_reshape(x, shape=(), **kw):
        shape = [x.shape[i] if s == 0 else s for i, s in enumerate(shape)]
        return x.reshape(shape)

    op("onnx_flatten")(lambda x, axis=1, **kw: x.reshape(int(torch.tensor(x.shape[:axis]).prod()) if axis else 1, -1))

    @op("onnx_unsqueeze")
    def onnx_unsqueeze(x, axes=(), **kw):
        for a in sorted(a % (x.dim() + len(axes)) for a in axes):
            x = x.unsqueeze(a)
        return x

    @op("onnx_batchnorm")
    def onnx_batchnorm(x, scale, bias, mean, var, epsilon=1e-5, **kw):
        shp = [1, -1] + [1] * (x.dim() - 2)
        return (x - mean.reshape(shp)) * (scale.reshape(shp) * torch.rsqrt(var.reshape(shp) + epsilon)) + bias.reshape(shp)

    @op("onnx_slice")
    def onnx_slice(x, starts=(), ends=(), axes=None, steps=None, **kw):
        axes = list(range(len(starts))) if axes is None else axes
        steps = [1] * len(starts) if steps is None else steps
        idx = [slice(None)] * x.dim()
        for s, e, a, st in zip(starts, ends, axes, steps):
            idx[a] = slice(s, None if e >= (1 << 62) else e, st)
        return x[tuple(idx)]


class OnnxFrameworkImporter:
    def __init__(self, trainable=True):
        self.trainable = trainable

    def runImport(self, path_or_bytes, dynamicVariables=None, suggestDynamicVariables=False):
        _register_helpers()
        if isinstance(path_or_bytes, (bytes, bytearray, memoryview)):
            data = path_or_bytes
        else:
            with open(path_or_bytes, "rb") as f:
                data = f.read()
        model = parse_model(data)
        unsupported = sorted({n["op"] for n in model["nodes"] if n["op"] not in OP_MAPPERS})
        if unsupported:
            raise NotImplementedError(f"ONNX import: no mapping rule for op types {unsupported}")
        sd = SameDiff.create()
        vars_, ctx = {}, {"consts": dict(model["initializers"])}
        consumed_as_const = set()
        for n in model["nodes"]:
            if n["op"] in ("Reshape", "Slice", "Squeeze", "Unsqueeze", "ReduceMean", "ReduceSum", "ReduceMax", "ReduceMin", "Clip"):
                consumed_as_const.update(i for i in n["inputs"][1:] if i)
        for name, t in model["initializers"].items():
            if name in consumed_as_const:
                continue
            if self.trainable and t.is_floating_point() and t.dim() >= 1:
                vars_[name] = sd.var(name, t.clone())
            else:
                vars_[name] = sd.constant(name, t.clone())
        for name, shape, elem in model["inputs"]:
            if name in model["initializers"]:
                continue
            dt = {1: DataType.FLOAT, 6: DataType.INT, 7: DataType.LONG, 10: DataType.HALF, 11: DataType.DOUBLE, 9: DataType.BOOL}.get(elem, DataType.FLOAT)
            vars_[name] = sd.placeHolder(name, dt, *(shape or []))
        for n in model["nodes"]:
            ins = [vars_.get(i) if i else None for i in n["inputs"]]
            out = OP_MAPPERS[n["op"]](sd, ctx, n, ins)
            outs = out if isinstance(out, (list, tuple)) else [out]
            for name, v in zip(n["outputs"], outs):
                if name and v.name != name:
                    v = sd.renameVariable(v.name, name) or sd.getVariable(name)
                vars_[name] = sd.getVariable(name) if sd.hasVariable(name) else v
        sd.metadata["onnx.outputs"] = ",".join(model["outputs"])
        sd.metadata["onnx.opset"] = str(model["opset"])
        self.outputs = model["outputs"]
        return sd


def importOnnx(path_or_bytes, trainable=True):
    return OnnxFrameworkImporter(trainable).runImport(path_or_bytes)
