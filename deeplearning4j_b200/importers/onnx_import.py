"""ONNX -> SameDiff import (``nd4j/samediff-import/samediff-import-onnx``: ``OnnxFrameworkImporter`` /
``ImportGraph`` with per-op mapping rules).  The ``.onnx`` file is parsed with the bundled protobuf wire reader, so
the ``onnx`` package is not required.  Initializers become SameDiff variables (constants when ``trainable=False``),
graph inputs become placeholders, and each node is mapped by an entry of ``OP_MAPPERS``; unknown ops raise with the
list of unsupported op types, as the reference's importer does."""
from __future__ import annotations

import math

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
    if typ == 5 or (typ == 0 and 6 in a):                            # GRAPH: the body of an If / Loop node
        return name, {"__graph__": parse_graph(a[6][0])}
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


def parse_graph(buf):
    g = pw.decode(buf)
    nodes = []
    for nb in g.get(1, []):
        n = pw.decode(nb)
        nodes.append({"inputs": [pw.string(s) for s in n.get(1, [])], "outputs": [pw.string(s) for s in n.get(2, [])],
                      "name": pw.string(n[3][0]) if 3 in n else "", "op": pw.string(n[4][0]),
                      "attrs": dict(parse_attribute(a) for a in n.get(5, []))})
    return {"nodes": nodes, "initializers": dict(parse_tensor(t) for t in g.get(5, [])), "inputs": [parse_value_info(v) for v in g.get(11, [])],
            "outputs": [parse_value_info(v)[0] for v in g.get(12, [])], "opset": 13}


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


# ----------------------------------------------------------------------------- control flow: If / Loop with sub-graphs
class _SubGraph:
    """A body graph of an If / Loop node imported into its own SameDiff.  Names that the body reads from the enclosing graph
    (ONNX sub-graphs see the outer scope) become placeholders and are handed in at every call."""

    def __init__(self, graph, trainable=False):
        produced = set(graph["initializers"]) | {i[0] for i in graph["inputs"]}
        for n in graph["nodes"]:
            produced.update(o for o in n["outputs"] if o)
        self.captured = []
        for n in graph["nodes"]:
            for i in _node_reads(n):
                if i and i not in produced and i not in self.captured:
                    self.captured.append(i)
        self.inputs = [i[0] for i in graph["inputs"] if i[0] not in graph["initializers"]]
        self.outputs = list(graph["outputs"])
        g = dict(graph)
        g["inputs"] = list(graph["inputs"]) + [(c, None, 1) for c in self.captured]
        self.sd = OnnxFrameworkImporter(trainable=False)._build(g)

    def run(self, inputs, captured):
        ph = dict(zip(self.inputs, inputs))
        ph.update(zip(self.captured, captured))
        known = {k: v for k, v in ph.items()}
        out = self.sd.output(known, *self.outputs)
        return [out[o].t if hasattr(out[o], "t") else out[o] for o in self.outputs]


def _node_reads(n):
    """Names a node reads, including what its own sub-graphs read from outside themselves."""
    reads = [i for i in n["inputs"] if i]
    for v in n["attrs"].values():
        if isinstance(v, dict) and "__graph__" in v:
            g = v["__graph__"]
            inner = set(g["initializers"]) | {i[0] for i in g["inputs"]}
            for m in g["nodes"]:
                inner.update(o for o in m["outputs"] if o)
            for m in g["nodes"]:
                reads += [i for i in _node_reads(m) if i not in inner]
    return reads


def _register_control_flow():
    from ..ops.registry import has, op
    if has("onnx.If"):
        return

    @op("onnx.If", n_out=-1, group="onnx_import")
    def onnx_if(cond, *captured, then_branch=None, else_branch=None, n_then=0, **kw):
        taken, caps = (then_branch, captured[:n_then]) if bool(cond.reshape(-1)[0]) else (else_branch, captured[n_then:])
        return tuple(taken.run([], caps))

    @op("onnx.Loop", n_out=-1, group="onnx_import")
    def onnx_loop(*args, body=None, n_carried=0, has_trip=True, has_cond=True, **kw):
        k = 0
        trip = None
        cond = True
        if has_trip:
            trip, k = int(args[0].reshape(-1)[0]), 1
        if has_cond:
            cond, k = bool(args[k].reshape(-1)[0]), k + 1
        carried = list(args[k:k + n_carried])
        captured = list(args[k + n_carried:])
        n_scan = len(body.outputs) - 1 - n_carried
        scans = [[] for _ in range(n_scan)]
        it = 0
        while cond and (trip is None or it < trip):
            outs = body.run([torch.tensor(it, dtype=torch.int64), torch.tensor(cond)] + carried, captured)
            cond = bool(outs[0].reshape(-1)[0])
            carried = list(outs[1:1 + n_carried])
            for s_, o in zip(scans, outs[1 + n_carried:]):
                s_.append(o)
            it += 1
            if it > 1_000_000:
                raise RuntimeError("onnx Loop: more than 1e6 iterations")
        return tuple(carried) + tuple(torch.stack(s_) if s_ else torch.zeros(0) for s_ in scans)


def _if(sd, ctx, n, x):
    tb, eb = _SubGraph(n["attrs"]["then_branch"]["__graph__"]), _SubGraph(n["attrs"]["else_branch"]["__graph__"])
    caps = [ctx["lookup"](c) for c in tb.captured] + [ctx["lookup"](c) for c in eb.captured]
    return sd._op("onnx.If", [x[0]] + caps, n_out=len(n["outputs"]), then_branch=tb, else_branch=eb, n_then=len(tb.captured))


def _loop(sd, ctx, n, x):
    body = _SubGraph(n["attrs"]["body"]["__graph__"])
    has_trip, has_cond = bool(n["inputs"][0]), len(n["inputs"]) > 1 and bool(n["inputs"][1])
    head = ([x[0]] if has_trip else []) + ([x[1]] if has_cond else [])
    carried = [v for v in x[2:]]
    caps = [ctx["lookup"](c) for c in body.captured]
    return sd._op("onnx.Loop", head + carried + caps, n_out=len(n["outputs"]), body=body, n_carried=len(carried), has_trip=has_trip, has_cond=has_cond)


OP_MAPPERS["If"] = _if
OP_MAPPERS["Loop"] = _loop


# ----------------------------------------------------------------------------- generic rules: ONNX semantics written once on tensors
def _ints(t):
    return [int(v) for v in (t.reshape(-1).tolist() if isinstance(t, torch.Tensor) else t)]


def _onnx_ops():
    """ONNX op type -> (function(inputs..., **attributes), number of outputs; -1 = one per declared output).  Inputs that ONNX passes
    as tensors (axes, shapes, pads, k, ...) stay tensor inputs of the graph node, so they may be computed at run time."""
    import torch.nn.functional as F

    def variadic(fn):
        def f(*xs, **kw):
            out = xs[0]
            for x in xs[1:]:
                out = fn(out, x)
            return out
        return f

    def red(fn):
        def f(x, axes_t=None, axes=None, keepdims=1, noop_with_empty_axes=0, **kw):
            ax = _ints(axes_t) if axes_t is not None else (list(axes) if axes is not None else None)
            if not ax:
                if noop_with_empty_axes and axes_t is not None:
                    return x
                ax = list(range(x.dim()))
            return fn(x, tuple(ax), bool(keepdims))
        return f

    def split(x, split_t=None, axis=0, split=None, num_outputs=None, **kw):
        sizes = _ints(split_t) if split_t is not None else (list(split) if split is not None else None)
        if sizes is None:
            k = int(num_outputs)
            step = -(-x.shape[axis] // k)
            return tuple(x.split(step, axis))
        return tuple(x.split(sizes, axis))

    def topk(x, k, axis=-1, largest=1, sorted=1, **kw):
        v, i = torch.topk(x, int(k.reshape(-1)[0]), dim=axis, largest=bool(largest), sorted=True)
        return v, i

    def pad(x, pads, value=None, axes=None, mode="constant", **kw):
        p = _ints(pads)
        ax = _ints(axes) if axes is not None else list(range(x.dim()))
        n = len(ax)
        lo, hi = [0] * x.dim(), [0] * x.dim()
        for j, a in enumerate(ax):
            lo[a % x.dim()], hi[a % x.dim()] = p[j], p[n + j]
        if mode == "constant":
            flat = []
            for d in reversed(range(x.dim())):
                flat += [lo[d], hi[d]]
            return F.pad(x, flat, value=float(value.reshape(-1)[0]) if value is not None and value.numel() else 0.0)
        y = x
        for d in range(x.dim()):
            if not (lo[d] or hi[d]):
                continue
            nd = y.shape[d]
            if mode == "reflect":
                front, back = y.narrow(d, 1, lo[d]).flip(d), y.narrow(d, nd - hi[d] - 1, hi[d]).flip(d)
            else:                                          # edge
                front = y.narrow(d, 0, 1).expand(*[lo[d] if k == d else s for k, s in enumerate(y.shape)])
                back = y.narrow(d, nd - 1, 1).expand(*[hi[d] if k == d else s for k, s in enumerate(y.shape)])
            y = torch.cat([front, y, back], d)
        return y

    def resize(x, roi=None, scales=None, sizes=None, mode="nearest", coordinate_transformation_mode="half_pixel", nearest_mode="round_prefer_floor", **kw):
        if sizes is not None and sizes.numel():
            out = _ints(sizes)[2:]
        else:
            sc = scales.reshape(-1).tolist()[2:]
            out = [int(math.floor(s * f)) for s, f in zip(x.shape[2:], sc)]
        if mode == "nearest":
            if coordinate_transformation_mode == "asymmetric" and nearest_mode == "floor":
                idx = [(torch.arange(o, device=x.device) * (s / o)).floor().long().clamp(max=s - 1) for o, s in zip(out, x.shape[2:])]
                y = x
                for d, i in enumerate(idx):
                    y = y.index_select(2 + d, i)
                return y
            return F.interpolate(x, size=out, mode="nearest-exact" if coordinate_transformation_mode in ("half_pixel", "pytorch_half_pixel") else "nearest")
        m = {1: "linear", 2: "bilinear", 3: "trilinear"}[len(out)] if mode == "linear" else "bicubic"
        return F.interpolate(x, size=out, mode=m, align_corners=coordinate_transformation_mode == "align_corners")

    def conv_t(x, w, b=None, strides=None, dilations=None, pads=None, output_padding=None, group=1, output_shape=None, auto_pad="NOTSET", **kw):
        nd = x.dim() - 2
        st, dl = list(strides or [1] * nd), list(dilations or [1] * nd)
        op_ = list(output_padding or [0] * nd)
        pd = list(pads or [0] * (2 * nd))
        fn = {1: F.conv_transpose1d, 2: F.conv_transpose2d, 3: F.conv_transpose3d}[nd]
        y = fn(x, w.to(x.dtype), None if b is None else b.to(x.dtype), st, 0, op_, group, dl)
        if output_shape is not None or auto_pad in ("SAME_UPPER", "SAME_LOWER"):
            tgt = list(output_shape) if output_shape is not None else [s * k for s, k in zip(x.shape[2:], st)]
            for d in range(nd):
                extra = y.shape[2 + d] - tgt[d]
                lo = extra // 2 if auto_pad != "SAME_LOWER" else extra - extra // 2
                y = y.narrow(2 + d, lo, tgt[d])
            return y
        for d in range(nd):
            y = y.narrow(2 + d, pd[d], y.shape[2 + d] - pd[d] - pd[nd + d])
        return y

    def inorm(x, scale, bias, epsilon=1e-5, **kw):
        return F.instance_norm(x, weight=scale, bias=bias, eps=float(epsilon))

    def lrn(x, size=5, alpha=1e-4, beta=0.75, bias=1.0, **kw):
        return F.local_response_norm(x, int(size), float(alpha), float(beta), float(bias))

    def d2s(x, blocksize=2, mode="DCR", **kw):
        n, c, h, w = x.shape
        b = int(blocksize)
        if mode == "DCR":
            return x.reshape(n, b, b, c // (b * b), h, w).permute(0, 3, 4, 1, 5, 2).reshape(n, c // (b * b), h * b, w * b)
        return x.reshape(n, c // (b * b), b, b, h, w).permute(0, 1, 4, 2, 5, 3).reshape(n, c // (b * b), h * b, w * b)

    def s2d(x, blocksize=2, **kw):
        n, c, h, w = x.shape
        b = int(blocksize)
        return x.reshape(n, c, h // b, b, w // b, b).permute(0, 3, 5, 1, 2, 4).reshape(n, c * b * b, h // b, w // b)

    def scatter_el(x, idx, upd, axis=0, reduction="none", **kw):
        idx = torch.where(idx < 0, idx + x.shape[axis], idx).long()
        if reduction == "none":
            return x.scatter(axis, idx, upd)
        return x.scatter_reduce(axis, idx, upd, {"add": "sum", "mul": "prod", "max": "amax", "min": "amin"}[reduction])

    def scatter_nd(x, idx, upd, reduction="none", **kw):
        y = x.clone()
        ix = tuple(idx.long()[..., i] for i in range(idx.shape[-1]))
        if reduction == "add":
            y.index_put_(ix, upd, accumulate=True)
        else:
            y[ix] = upd
        return y

    def gather_nd(x, idx, batch_dims=0, **kw):
        idx = idx.long()
        if batch_dims:
            return torch.stack([gather_nd(xb, ib, batch_dims - 1) for xb, ib in zip(x, idx)])
        return x[tuple(idx[..., i] for i in range(idx.shape[-1]))]

    def onehot(idx, depth, values, axis=-1, **kw):
        d = int(depth.reshape(-1)[0])
        i = idx.long()
        i = torch.where(i < 0, i + d, i)
        oh = F.one_hot(i.clamp(0, d - 1), d).bool() & ((i >= 0) & (i < d)).unsqueeze(-1)
        y = torch.where(oh, values[1], values[0])
        return y if axis in (-1, idx.dim()) else y.movedim(-1, axis)

    def cumsum(x, axis, exclusive=0, reverse=0, **kw):
        a = int(axis.reshape(-1)[0])
        if reverse:
            x = x.flip(a)
        y = x.cumsum(a)
        if exclusive:
            y = y - x
        return y.flip(a) if reverse else y

    def arg(fn):
        def f(x, axis=0, keepdims=1, select_last_index=0, **kw):
            if select_last_index:
                r = x.shape[axis] - 1 - fn(x.flip(axis), axis, bool(keepdims))
                return r
            return fn(x, axis, bool(keepdims))
        return f

    def lstm(X, W, R, B=None, seq_lens=None, h0=None, c0=None, P=None, hidden_size=None, direction="forward", **kw):
        """ONNX LSTM (gate order i, o, f, c; layout 0): X [T, N, I] -> Y [T, D, N, H], Y_h, Y_c [D, N, H]."""
        T, N, _ = X.shape
        D, H = W.shape[0], R.shape[2]
        ys, hs, cs = [], [], []
        for d in range(D):
            w, r = W[d], R[d]
            b = (B[d][:4 * H] + B[d][4 * H:]) if B is not None else X.new_zeros(4 * H)
            h = h0[d] if h0 is not None else X.new_zeros(N, H)
            c = c0[d] if c0 is not None else X.new_zeros(N, H)
            steps = range(T - 1, -1, -1) if (direction == "reverse" or d == 1) else range(T)
            out = [None] * T
            for t in steps:
                z = X[t] @ w.t() + h @ r.t() + b
                i, o, f, g = z[:, :H], z[:, H:2 * H], z[:, 2 * H:3 * H], z[:, 3 * H:]
                if P is not None:
                    i, f = i + P[d][:H] * c, f + P[d][2 * H:] * c
                i, f = torch.sigmoid(i), torch.sigmoid(f)
                c = f * c + i * torch.tanh(g)
                if P is not None:
                    o = o + P[d][H:2 * H] * c
                h = torch.sigmoid(o) * torch.tanh(c)
                out[t] = h
            ys.append(torch.stack(out))
            hs.append(h)
            cs.append(c)
        return torch.stack(ys, 1), torch.stack(hs), torch.stack(cs)

    def gru(X, W, R, B=None, seq_lens=None, h0=None, hidden_size=None, direction="forward", linear_before_reset=0, **kw):
        """ONNX GRU (gate order z, r, h): X [T, N, I] -> Y [T, D, N, H], Y_h [D, N, H]."""
        T, N, _ = X.shape
        D, H = W.shape[0], R.shape[2]
        ys, hs = [], []
        for d in range(D):
            w, r = W[d], R[d]
            wb = B[d][:3 * H] if B is not None else X.new_zeros(3 * H)
            rb = B[d][3 * H:] if B is not None else X.new_zeros(3 * H)
            h = h0[d] if h0 is not None else X.new_zeros(N, H)
            steps = range(T - 1, -1, -1) if (direction == "reverse" or d == 1) else range(T)
            out = [None] * T
            for t in steps:
                xz = X[t] @ w.t() + wb
                z = torch.sigmoid(xz[:, :H] + h @ r[:H].t() + rb[:H])
                rr = torch.sigmoid(xz[:, H:2 * H] + h @ r[H:2 * H].t() + rb[H:2 * H])
                if linear_before_reset:
                    hh = torch.tanh(xz[:, 2 * H:] + rr * (h @ r[2 * H:].t() + rb[2 * H:]))
                else:
                    hh = torch.tanh(xz[:, 2 * H:] + (rr * h) @ r[2 * H:].t() + rb[2 * H:])
                h = (1 - z) * hh + z * h
                out[t] = h
            ys.append(torch.stack(out))
            hs.append(h)
        return torch.stack(ys, 1), torch.stack(hs)

    def rnn(x, w, r, b=None, seq_lens=None, h0=None, hidden_size=None, direction="forward", activations=None, **kw):
        """Elman RNN: h_t = f(x_t W^T + h_{t-1} R^T + Wb + Rb); Y [T, dirs, N, H], Y_h [dirs, N, H]."""
        T_, N = x.shape[0], x.shape[1]
        dirs = w.shape[0]
        H = w.shape[1]
        acts = [a.decode() if isinstance(a, bytes) else a for a in (activations or ["Tanh"] * dirs)]
        fmap = {"Tanh": torch.tanh, "Relu": torch.relu, "Sigmoid": torch.sigmoid}
        ys, hs = [], []
        for d in range(dirs):
            f = fmap[acts[d] if d < len(acts) else acts[0]]
            h = h0[d] if h0 is not None else x.new_zeros(N, H)
            bias = (b[d, :H] + b[d, H:]) if b is not None else 0
            order = range(T_ - 1, -1, -1) if (direction == "reverse" or d == 1) else range(T_)
            out = [None] * T_
            for t in order:
                h = f(x[t] @ w[d].t() + h @ r[d].t() + bias)
                out[t] = h
            ys.append(torch.stack(out, 0))
            hs.append(h)
        return torch.stack(ys, 1), torch.stack(hs, 0)

    def _bcast_axis(t, like, axis):
        if t.dim() == 0 or t.numel() == 1:
            return t.reshape(())
        shp = [1] * like.dim()
        shp[axis] = -1
        return t.reshape(shp)

    def quantize_linear(x, scale, zp=None, axis=1, saturate=1, **kw):
        dt = zp.dtype if zp is not None else torch.uint8
        lo, hi = (0, 255) if dt == torch.uint8 else (-128, 127)
        z = _bcast_axis(zp, x, axis).to(x.dtype) if zp is not None else 0
        return (torch.round(x / _bcast_axis(scale, x, axis)) + z).clamp(lo, hi).to(dt)

    def dequantize_linear(x, scale, zp=None, axis=1, **kw):
        z = _bcast_axis(zp, x, axis).to(scale.dtype) if zp is not None else 0
        return (x.to(scale.dtype) - z) * _bcast_axis(scale, x, axis)

    def reverse_sequence(x, lens, batch_axis=1, time_axis=0, **kw):
        y = x.clone()
        for bi, L in enumerate(_ints(lens)):
            sl = [slice(None)] * x.dim()
            sl[batch_axis] = bi
            sl[time_axis] = slice(0, L)
            seg = x[tuple(sl)]
            ax = time_axis - (1 if batch_axis < time_axis else 0)
            y[tuple(sl)] = seg.flip(ax)
        return y

    def unique(x, axis=None, sorted=1, **kw):
        """Y, first indices, inverse indices, counts (sorted order; ONNX's unsorted order = first occurrence, restored below)."""
        flat = x.reshape(-1) if axis is None else x
        y, inv, cnt = torch.unique(flat, sorted=True, return_inverse=True, return_counts=True, dim=None if axis is None else axis)
        n = y.shape[0] if axis is None else y.shape[axis]
        inv1 = inv.reshape(-1)
        first = torch.full((n,), inv1.numel(), dtype=torch.int64)
        first.scatter_reduce_(0, inv1, torch.arange(inv1.numel()), reduce="amin")
        if not sorted:
            order = first.argsort()
            y = y.index_select(0 if axis is None else axis, order)
            rank = torch.empty_like(order)
            rank[order] = torch.arange(n)
            inv, cnt, first = rank[inv], cnt[order], first[order]
        return y, first, inv, cnt

    def nms(boxes, scores, max_out=None, iou_thr=None, score_thr=None, center_point_box=0, **kw):
        """[num_selected, 3] rows (batch, class, box index), greedy per batch and class in order of decreasing score."""
        m = int(max_out.reshape(-1)[0]) if max_out is not None and max_out.numel() else 0
        it = float(iou_thr.reshape(-1)[0]) if iou_thr is not None and iou_thr.numel() else 0.0
        st = float(score_thr.reshape(-1)[0]) if score_thr is not None and score_thr.numel() else None
        sel = []
        if m == 0:
            return torch.zeros((0, 3), dtype=torch.int64)
        for bi in range(boxes.shape[0]):
            bx = boxes[bi]
            if center_point_box:
                cx, cy, w_, h_ = bx.unbind(1)
                x1, y1, x2, y2 = cx - w_ / 2, cy - h_ / 2, cx + w_ / 2, cy + h_ / 2
            else:
                y1, x1, y2, x2 = bx.unbind(1)
                x1, x2 = torch.minimum(x1, x2), torch.maximum(x1, x2)
                y1, y2 = torch.minimum(y1, y2), torch.maximum(y1, y2)
            area = (x2 - x1) * (y2 - y1)
            for ci in range(scores.shape[1]):
                sc = scores[bi, ci]
                order = sc.argsort(descending=True).tolist()
                keep = []
                for i in order:
                    if st is not None and float(sc[i]) <= st:
                        break
                    ok = True
                    for j in keep:
                        iw = (torch.minimum(x2[i], x2[j]) - torch.maximum(x1[i], x1[j])).clamp(min=0)
                        ih = (torch.minimum(y2[i], y2[j]) - torch.maximum(y1[i], y1[j])).clamp(min=0)
                        inter = iw * ih
                        union = area[i] + area[j] - inter
                        if float(union) > 0 and float(inter / union) > it:
                            ok = False
                            break
                    if ok:
                        keep.append(i)
                        sel.append([bi, ci, i])
                        if len(keep) >= m:
                            break
        return torch.tensor(sel, dtype=torch.int64).reshape(-1, 3)

    def roi_align(x, rois, batch_idx, mode="avg", output_height=1, output_width=1, sampling_ratio=0, spatial_scale=1.0,
                  coordinate_transformation_mode="half_pixel", **kw):
        mode = mode.decode() if isinstance(mode, bytes) else mode
        ctm = coordinate_transformation_mode.decode() if isinstance(coordinate_transformation_mode, bytes) else coordinate_transformation_mode
        off = 0.5 if ctm == "half_pixel" else 0.0
        N, C, H, W = x.shape
        out = x.new_zeros(rois.shape[0], C, output_height, output_width)
        for r in range(rois.shape[0]):
            x1, y1, x2, y2 = [float(v) * spatial_scale - off for v in rois[r].tolist()]
            rw, rh = x2 - x1, y2 - y1
            if ctm != "half_pixel":
                rw, rh = max(rw, 1.0), max(rh, 1.0)
            bw, bh = rw / output_width, rh / output_height
            sx = sampling_ratio if sampling_ratio > 0 else max(1, int(-(-rw // output_width)))
            sy = sampling_ratio if sampling_ratio > 0 else max(1, int(-(-rh // output_height)))
            img = x[int(batch_idx[r])]
            for ph in range(output_height):
                for pw_ in range(output_width):
                    vals = []
                    for iy in range(sy):
                        yy = y1 + ph * bh + (iy + 0.5) * bh / sy
                        for ix in range(sx):
                            xx = x1 + pw_ * bw + (ix + 0.5) * bw / sx
                            if yy < -1.0 or yy > H or xx < -1.0 or xx > W:
                                vals.append(x.new_zeros(C))
                                continue
                            yc, xc = min(max(yy, 0.0), H - 1), min(max(xx, 0.0), W - 1)
                            y0, x0 = int(yc), int(xc)
                            y1i, x1i = min(y0 + 1, H - 1), min(x0 + 1, W - 1)
                            ly, lx = yc - y0, xc - x0
                            vals.append(img[:, y0, x0] * (1 - ly) * (1 - lx) + img[:, y0, x1i] * (1 - ly) * lx
                                        + img[:, y1i, x0] * ly * (1 - lx) + img[:, y1i, x1i] * ly * lx)
                    v = torch.stack(vals, 0)
                    out[r, :, ph, pw_] = v.mean(0) if mode == "avg" else v.max(0).values
        return out

    T = {
        "Less": (lambda a, b, **k: a < b, 1), "LessOrEqual": (lambda a, b, **k: a <= b, 1), "Greater": (lambda a, b, **k: a > b, 1),
        "GreaterOrEqual": (lambda a, b, **k: a >= b, 1), "Equal": (lambda a, b, **k: a == b, 1), "Not": (lambda a, **k: ~a, 1),
        "And": (lambda a, b, **k: a & b, 1), "Or": (lambda a, b, **k: a | b, 1), "Xor": (lambda a, b, **k: a ^ b, 1),
        "Where": (lambda c, a, b, **k: torch.where(c, a, b), 1),
        "Max": (variadic(torch.maximum), 1), "Min": (variadic(torch.minimum), 1), "Sum": (variadic(torch.add), 1),
        "Mean": (lambda *xs, **k: variadic(torch.add)(*xs) / len(xs), 1),
        "Sin": (lambda x, **k: x.sin(), 1), "Cos": (lambda x, **k: x.cos(), 1), "Tan": (lambda x, **k: x.tan(), 1), "Asin": (lambda x, **k: x.asin(), 1),
        "Acos": (lambda x, **k: x.acos(), 1), "Atan": (lambda x, **k: x.atan(), 1), "Sinh": (lambda x, **k: x.sinh(), 1), "Cosh": (lambda x, **k: x.cosh(), 1),
        "Asinh": (lambda x, **k: x.asinh(), 1), "Acosh": (lambda x, **k: x.acosh(), 1), "Atanh": (lambda x, **k: x.atanh(), 1),
        "Round": (lambda x, **k: x.round(), 1), "Sign": (lambda x, **k: x.sign(), 1), "Softsign": (lambda x, **k: x / (1 + x.abs()), 1),
        "Selu": (lambda x, alpha=1.6732632423543772, gamma=1.0507009873554805, **k: gamma * torch.where(x > 0, x, alpha * x.expm1()), 1),
        "HardSigmoid": (lambda x, alpha=0.2, beta=0.5, **k: (alpha * x + beta).clamp(0, 1), 1),
        "HardSwish": (lambda x, **k: x * (x / 6 + 0.5).clamp(0, 1), 1), "PRelu": (lambda x, s, **k: torch.where(x >= 0, x, x * s), 1),
        "ThresholdedRelu": (lambda x, alpha=1.0, **k: torch.where(x > alpha, x, torch.zeros_like(x)), 1),
        "Mish": (lambda x, **k: x * torch.tanh(F.softplus(x)), 1), "Celu": (lambda x, alpha=1.0, **k: F.celu(x, alpha), 1),
        "IsNaN": (lambda x, **k: x.isnan(), 1), "IsInf": (lambda x, detect_negative=1, detect_positive=1, **k:
                                                          (x.isposinf() if detect_positive else torch.zeros_like(x, dtype=torch.bool)) |
                                                          (x.isneginf() if detect_negative else torch.zeros_like(x, dtype=torch.bool)), 1),
        "Expand": (lambda x, sh, **k: x.broadcast_to(torch.broadcast_shapes(tuple(x.shape), tuple(_ints(sh)))), 1),
        "Tile": (lambda x, r, **k: x.repeat(*_ints(r)), 1),
        "Range": (lambda a, b, c, **k: torch.arange(a.item(), b.item(), c.item(), dtype=a.dtype, device=a.device), 1),
        "ConstantOfShape": (lambda sh, value=None, **k: torch.full(_ints(sh), (value.reshape(-1)[0].item() if value is not None else 0.0),
                                                                  dtype=value.dtype if value is not None else torch.float32), 1),
        "Split": (split, -1), "TopK": (topk, 2),
        "ArgMax": (arg(lambda x, a, kd: x.argmax(a, kd)), 1), "ArgMin": (arg(lambda x, a, kd: x.argmin(a, kd)), 1),
        "CumSum": (cumsum, 1), "OneHot": (onehot, 1),
        "GatherElements": (lambda x, i, axis=0, **k: x.gather(axis, torch.where(i < 0, i + x.shape[axis], i).long()), 1),
        "GatherND": (gather_nd, 1), "ScatterElements": (scatter_el, 1), "Scatter": (scatter_el, 1), "ScatterND": (scatter_nd, 1),
        "Pad": (pad, 1), "Resize": (resize, 1), "Upsample": (lambda x, scales, mode="nearest", **k: resize(x, None, scales, None, mode, "asymmetric", "floor"), 1),
        "DepthToSpace": (d2s, 1), "SpaceToDepth": (s2d, 1), "ConvTranspose": (conv_t, 1), "InstanceNormalization": (inorm, 1), "LRN": (lrn, 1),
        "ReduceProd": (red(lambda x, ax, kd: [x := x.prod(d, keepdim=True) for d in ax][-1] if kd else
                           [x := x.prod(d) for d in sorted((a % x.dim() for a in ax), reverse=True)][-1]), 1),
        "ReduceL1": (red(lambda x, ax, kd: x.abs().sum(ax, kd)), 1), "ReduceL2": (red(lambda x, ax, kd: x.pow(2).sum(ax, kd).sqrt()), 1),
        "ReduceLogSumExp": (red(lambda x, ax, kd: x.logsumexp(ax, kd)), 1), "ReduceSumSquare": (red(lambda x, ax, kd: x.pow(2).sum(ax, kd)), 1),
        "ReduceLogSum": (red(lambda x, ax, kd: x.sum(ax, kd).log()), 1),
        "Einsum": (lambda *xs, equation="", **k: torch.einsum(equation, *xs), 1), "NonZero": (lambda x, **k: x.nonzero().t(), 1),
        "Size": (lambda x, **k: torch.tensor(x.numel(), dtype=torch.int64), 1),
        "Trilu": (lambda x, kk=None, upper=1, **k: (torch.triu if upper else torch.tril)(x, int(kk.reshape(-1)[0]) if kk is not None else 0), 1),
        "Mod": (lambda a, b, fmod=0, **k: torch.fmod(a, b) if fmod else torch.remainder(a, b), 1),
        "BitShift": (lambda a, b, direction="LEFT", **k: a << b if direction == "LEFT" else a >> b, 1),
        "EyeLike": (lambda x, k=0, **kw: torch.eye(x.shape[0], x.shape[1], dtype=x.dtype).roll(int(k), 1) if not k else torch.diag(torch.ones(min(x.shape[0], x.shape[1] - k) if k > 0 else min(x.shape[0] + k, x.shape[1]), dtype=x.dtype), int(k))[:x.shape[0], :x.shape[1]], 1),
        "Hardmax": (lambda x, axis=-1, **k: F.one_hot(x.argmax(axis), x.shape[axis]).to(x.dtype).movedim(-1, axis), 1),
        "LpNormalization": (lambda x, axis=-1, p=2, **k: x / x.norm(p=p, dim=axis, keepdim=True), 1),
        "MeanVarianceNormalization": (lambda x, axes=(0, 2, 3), **k: (x - x.mean(tuple(axes), keepdim=True)) / x.var(tuple(axes), unbiased=False, keepdim=True).sqrt(), 1),
        "GlobalLpPool": (lambda x, p=2, **k: x.norm(p=p, dim=tuple(range(2, x.dim())), keepdim=True), 1),
        "Sqrt": (lambda x, **k: x.sqrt(), 1),
        "LSTM": (lstm, 3), "GRU": (gru, 2), "RNN": (rnn, 2),
        "Compress": (lambda x, cond, axis=None, **k: (x.reshape(-1)[:cond.numel()][cond.reshape(-1).bool()] if axis is None
                                                     else x.index_select(axis, cond.reshape(-1).bool().nonzero().reshape(-1))), 1),
        "Det": (lambda x, **k: torch.linalg.det(x), 1),
        "Shrink": (lambda x, bias=0.0, lambd=0.5, **k: torch.where(x < -lambd, x + bias, torch.where(x > lambd, x - bias, torch.zeros_like(x))), 1),
        "GroupNormalization": (lambda x, scale, b, num_groups=1, epsilon=1e-5, **k: F.group_norm(
            x, int(num_groups), scale if scale.numel() == x.shape[1] else scale.repeat_interleave(x.shape[1] // scale.numel()),
            b if b.numel() == x.shape[1] else b.repeat_interleave(x.shape[1] // b.numel()), epsilon), 1),
        "QuantizeLinear": (quantize_linear, 1), "DequantizeLinear": (dequantize_linear, 1),
        "ReverseSequence": (reverse_sequence, 1), "Unique": (unique, 4),
        "NonMaxSuppression": (nms, 1), "RoiAlign": (roi_align, 1),
    }
    T.update(_onnx_ops_more())
    return T


def _onnx_ops_more():
    """Second table: integer / quantised linear algebra, window and spectral ops, random ops, losses, unpooling, grid sampling."""
    import math
    import torch.nn.functional as F
    TORCH_DT = {1: torch.float32, 2: torch.uint8, 3: torch.int8, 5: torch.int16, 6: torch.int32, 7: torch.int64, 9: torch.bool, 10: torch.float16,
                11: torch.float64, 16: torch.bfloat16}

    def window(kind):
        def f(size, output_datatype=1, periodic=1, **kw):
            n = int(size)
            N = n if periodic else n - 1
            k = torch.arange(n, dtype=torch.float64)
            if kind == "hann":
                w = 0.5 - 0.5 * torch.cos(2 * math.pi * k / N)
            elif kind == "hamming":
                w = 25 / 46 - 21 / 46 * torch.cos(2 * math.pi * k / N)
            else:
                w = 0.42 - 0.5 * torch.cos(2 * math.pi * k / N) + 0.08 * torch.cos(4 * math.pi * k / N)
            return w.to(TORCH_DT[int(output_datatype)])
        return f

    def pads_of(x, kshape, strides, dilations, pads, auto_pad):
        nd = len(kshape)
        auto_pad = auto_pad.decode() if isinstance(auto_pad, bytes) else auto_pad
        if auto_pad in ("SAME_UPPER", "SAME_LOWER"):
            out = []
            for d in range(nd):
                total = max((-(-x.shape[2 + d] // strides[d]) - 1) * strides[d] + (kshape[d] - 1) * dilations[d] + 1 - x.shape[2 + d], 0)
                lo = total // 2 if auto_pad == "SAME_UPPER" else total - total // 2
                out.append((lo, total - lo))
            return out
        pads = list(pads) if pads is not None else [0] * (2 * nd)
        return [(pads[d], pads[d + nd]) for d in range(nd)]

    def conv_int(x, w, x_zp=None, w_zp=None, strides=None, dilations=None, pads=None, group=1, auto_pad="NOTSET", kernel_shape=None, **kw):
        nd = w.dim() - 2
        strides, dilations = list(strides or [1] * nd), list(dilations or [1] * nd)
        xf = x.to(torch.float64) - (x_zp.to(torch.float64) if x_zp is not None else 0)
        wz = w_zp.to(torch.float64).reshape(-1, *([1] * (w.dim() - 1))) if w_zp is not None and w_zp.numel() > 1 else (w_zp.to(torch.float64) if w_zp is not None else 0)
        wf = w.to(torch.float64) - wz
        pp = pads_of(x, list(w.shape[2:]), strides, dilations, pads, auto_pad)
        flat = [v for lo_hi in reversed(pp) for v in lo_hi]
        xf = F.pad(xf, flat)
        conv = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[nd]
        return conv(xf, wf, None, strides, 0, dilations, int(group))

    def qlinear_conv(x, xs, xz, w, ws, wz, ys, yz, b=None, **kw):
        acc = conv_int(x, w, xz, wz, **kw)
        scale = (xs.double() * ws.double()).reshape(1, -1, *([1] * (acc.dim() - 2))) if ws.numel() > 1 else xs.double() * ws.double()
        if b is not None:
            acc = acc + b.double().reshape(1, -1, *([1] * (acc.dim() - 2)))
        info = torch.iinfo(yz.dtype)
        return torch.clamp(torch.round(acc * scale / ys.double()) + yz.double(), info.min, info.max).to(yz.dtype)

    def matmul_int(a, b, a_zp=None, b_zp=None, **kw):
        af = a.to(torch.int64) - (a_zp.to(torch.int64).reshape(-1, 1) if a_zp is not None and a_zp.numel() > 1 else (a_zp.to(torch.int64) if a_zp is not None else 0))
        bf = b.to(torch.int64) - (b_zp.to(torch.int64) if b_zp is not None else 0)
        return (af.double() @ bf.double()).to(torch.int32)

    def qlinear_matmul(a, as_, az, b, bs, bz, ys, yz, **kw):
        acc = (a.double() - az.double()) @ (b.double() - bz.double())
        info = torch.iinfo(yz.dtype)
        return torch.clamp(torch.round(acc * as_.double() * bs.double() / ys.double()) + yz.double(), info.min, info.max).to(yz.dtype)

    def dyn_quant(x, **kw):
        lo, hi = min(float(x.min()), 0.0), max(float(x.max()), 0.0)
        scale = (hi - lo) / 255.0 or 1.0
        zp = max(0.0, min(255.0, round(-lo / scale)))                                   # Python rounds half to even, as the specification asks
        y = torch.clamp(torch.round(x / scale) + zp, 0, 255).to(torch.uint8)
        return y, torch.tensor(scale, dtype=torch.float32), torch.tensor(zp, dtype=torch.uint8)

    def lp_pool(x, kernel_shape=None, strides=None, pads=None, p=2, auto_pad="NOTSET", dilations=None, ceil_mode=0, **kw):
        nd = len(kernel_shape)
        strides, dilations = list(strides or [1] * nd), list(dilations or [1] * nd)
        pp = pads_of(x, list(kernel_shape), strides, dilations, pads, auto_pad)
        xp = F.pad(x.abs() ** p, [v for lo_hi in reversed(pp) for v in lo_hi])
        pool = {1: F.avg_pool1d, 2: F.avg_pool2d, 3: F.avg_pool3d}[nd]
        return (pool(xp, list(kernel_shape), strides, 0, bool(ceil_mode)) * float(np.prod(kernel_shape))) ** (1.0 / p)

    def max_unpool(x, idx, output_shape=None, kernel_shape=None, strides=None, pads=None, **kw):
        nd = len(kernel_shape)
        strides = list(strides or [1] * nd)
        pads = list(pads or [0] * (2 * nd))
        if output_shape is not None:
            shape = _ints(output_shape)
        else:
            shape = list(x.shape[:2]) + [(x.shape[2 + d] - 1) * strides[d] + kernel_shape[d] - pads[d] - pads[d + nd] for d in range(nd)]
        out = torch.zeros(int(np.prod(shape)), dtype=x.dtype)
        out[idx.reshape(-1).long()] = x.reshape(-1)                                      # indices are flat offsets into the whole output tensor
        return out.reshape(shape)

    def max_roi_pool(x, rois, pooled_shape=None, spatial_scale=1.0, **kw):
        ph, pw = pooled_shape
        out = []
        for r in rois:
            b = int(r[0])
            x1, y1, x2, y2 = [int(round(float(v) * spatial_scale)) for v in r[1:]]
            h, w = max(y2 - y1 + 1, 1), max(x2 - x1 + 1, 1)
            cell = torch.full((x.shape[1], ph, pw), 0.0, dtype=x.dtype)
            for i in range(ph):
                for j in range(pw):
                    ys, ye = y1 + int(math.floor(i * h / ph)), y1 + int(math.ceil((i + 1) * h / ph))
                    xs, xe = x1 + int(math.floor(j * w / pw)), x1 + int(math.ceil((j + 1) * w / pw))
                    ys, ye, xs, xe = max(ys, 0), min(ye, x.shape[2]), max(xs, 0), min(xe, x.shape[3])
                    if ye > ys and xe > xs:
                        cell[:, i, j] = x[b, :, ys:ye, xs:xe].amax((1, 2))
            out.append(cell)
        return torch.stack(out)

    def grid_sample(x, grid, mode="linear", padding_mode="zeros", align_corners=0, **kw):
        dec = lambda v: v.decode() if isinstance(v, bytes) else v
        mode = {"linear": "bilinear", "bilinear": "bilinear", "nearest": "nearest", "cubic": "bicubic", "bicubic": "bicubic"}[dec(mode)]
        return F.grid_sample(x, grid.to(x.dtype), mode=mode, padding_mode=dec(padding_mode), align_corners=bool(align_corners))

    def col2im(cols, image_shape, block_shape, dilations=None, pads=None, strides=None, **kw):
        img, blk = _ints(image_shape), _ints(block_shape)
        nd = len(img)
        if nd != 2:
            raise NotImplementedError("Col2Im for other than two spatial axes")
        pads = list(pads or [0] * 4)
        if pads[0] != pads[2] or pads[1] != pads[3]:
            raise NotImplementedError("Col2Im with different begin and end pads")
        return F.fold(cols, img, blk, list(dilations or [1, 1]), pads[:2], list(strides or [1, 1]))

    def center_crop_pad(x, shape, axes=None, **kw):
        tgt = _ints(shape)
        axes = list(axes) if axes is not None else list(range(x.dim()))
        for a, t in zip(axes, tgt):
            a = a % x.dim()
            cur = x.shape[a]
            if cur > t:
                x = x.narrow(a, (cur - t) // 2, t)
            elif cur < t:
                lo = (t - cur) // 2
                pad = [0, 0] * x.dim()
                pad[2 * (x.dim() - 1 - a)], pad[2 * (x.dim() - 1 - a) + 1] = lo, t - cur - lo
                x = F.pad(x, pad)
        return x

    def nll_loss(x, target, weight=None, ignore_index=None, reduction="mean", **kw):
        reduction = reduction.decode() if isinstance(reduction, bytes) else reduction
        return F.nll_loss(x, target.long(), weight, ignore_index=-100 if ignore_index is None else int(ignore_index), reduction=reduction)

    def sce_loss(scores, labels, weights=None, ignore_index=None, reduction="mean", **kw):
        reduction = reduction.decode() if isinstance(reduction, bytes) else reduction
        logp = F.log_softmax(scores, 1)
        return F.nll_loss(logp, labels.long(), weights, ignore_index=-100 if ignore_index is None else int(ignore_index), reduction=reduction), logp

    def dft(x, dft_length=None, axis=None, inverse=0, onesided=0, **kw):
        ax = int(axis) if axis is not None else -2
        ax = ax % x.dim()
        n = int(dft_length) if dft_length is not None else None
        z = torch.view_as_complex(x.contiguous()) if x.shape[-1] == 2 else x[..., 0].to(torch.complex64 if x.dtype != torch.float64 else torch.complex128)
        if inverse:
            y = torch.fft.ifft(z, n=n, dim=ax)
        elif onesided:
            if x.shape[-1] != 1:
                raise ValueError("a one-sided DFT needs a real input")
            y = torch.fft.rfft(x[..., 0], n=n, dim=ax)
        else:
            y = torch.fft.fft(z, n=n, dim=ax)
        return torch.view_as_real(y)

    def stft(signal, frame_step, window=None, frame_length=None, onesided=1, **kw):
        step = int(frame_step)
        n = int(frame_length) if frame_length is not None else window.numel()
        sig = signal[..., 0] if signal.shape[-1] == 1 else torch.view_as_complex(signal.contiguous())
        frames = sig.unfold(1, n, step)                                                  # [batch, frames, n]
        if window is not None:
            frames = frames * window.to(frames.dtype if not frames.is_complex() else window.dtype)
        y = torch.fft.rfft(frames, dim=-1) if onesided and not frames.is_complex() else torch.fft.fft(frames, dim=-1)
        return torch.view_as_real(y)

    def mel_weights(num_mel_bins, dft_length, sample_rate, lower_edge_hertz, upper_edge_hertz, output_datatype=1, **kw):
        nb, n, sr = int(num_mel_bins), int(dft_length), int(sample_rate)
        lo, hi = float(lower_edge_hertz), float(upper_edge_hertz)
        mel = lambda f: 2595.0 * math.log10(1.0 + f / 700.0)
        pts = [lo_m for lo_m in np.linspace(mel(lo), mel(hi), nb + 2)]
        bins = [int(math.floor((n + 1) * (700.0 * (10 ** (m / 2595.0) - 1.0)) / sr)) for m in pts]
        out = torch.zeros(n // 2 + 1, nb, dtype=torch.float64)
        for i in range(nb):
            l, c, r = bins[i], bins[i + 1], bins[i + 2]
            if c == l:
                out[c, i] = 1.0
            else:
                for j in range(l, c + 1):
                    out[j, i] = (j - l) / (c - l)
            for j in range(c + 1, r):
                out[j, i] = (r - j) / (r - c)
        return out.to(TORCH_DT[int(output_datatype)])

    def rnd(kind, like):
        def f(*xs, shape=None, dtype=None, mean=0.0, scale=1.0, low=0.0, high=1.0, seed=None, **kw):
            shp = list(xs[0].shape) if like else [int(v) for v in shape]
            dt = TORCH_DT[int(dtype)] if dtype is not None else (xs[0].dtype if like and xs[0].dtype.is_floating_point else torch.float32)
            gen = torch.Generator().manual_seed(int(seed)) if seed is not None else None
            if kind == "normal":
                return (torch.randn(shp, generator=gen) * scale + mean).to(dt)
            return (torch.rand(shp, generator=gen) * (high - low) + low).to(dt)
        return f

    return {
        "BitwiseAnd": (lambda a, b, **k: a & b, 1), "BitwiseOr": (lambda a, b, **k: a | b, 1), "BitwiseXor": (lambda a, b, **k: a ^ b, 1),
        "BitwiseNot": (lambda a, **k: ~a, 1),
        "CastLike": (lambda x, like, **k: x.to(like.dtype), 1),
        "HannWindow": (window("hann"), 1), "HammingWindow": (window("hamming"), 1), "BlackmanWindow": (window("blackman"), 1),
        "ConvInteger": (lambda x, w, xz=None, wz=None, **k: conv_int(x, w, xz, wz, **k).to(torch.int32), 1),
        "MatMulInteger": (matmul_int, 1), "QLinearConv": (qlinear_conv, 1), "QLinearMatMul": (qlinear_matmul, 1),
        "DynamicQuantizeLinear": (dyn_quant, 3),
        "LpPool": (lp_pool, 1), "MaxUnpool": (max_unpool, 1), "MaxRoiPool": (max_roi_pool, 1), "GridSample": (grid_sample, 1),
        "Col2Im": (col2im, 1), "CenterCropPad": (center_crop_pad, 1),
        "NegativeLogLikelihoodLoss": (nll_loss, 1), "SoftmaxCrossEntropyLoss": (sce_loss, -1),
        "DFT": (dft, 1), "STFT": (stft, 1), "MelWeightMatrix": (mel_weights, 1),
        "RandomNormal": (rnd("normal", False), 1), "RandomNormalLike": (rnd("normal", True), 1),
        "RandomUniform": (rnd("uniform", False), 1), "RandomUniformLike": (rnd("uniform", True), 1),
        "Bernoulli": (lambda x, dtype=None, seed=None, **k: torch.bernoulli(x.float(), generator=torch.Generator().manual_seed(int(seed)) if seed is not None else None)
                      .to(TORCH_DT[int(dtype)] if dtype is not None else x.dtype), 1),
        "Multinomial": (lambda x, sample_size=1, dtype=6, seed=None, **k: torch.multinomial(
            x.float().softmax(-1), int(sample_size), True, generator=torch.Generator().manual_seed(int(seed)) if seed is not None else None).to(TORCH_DT[int(dtype)]), 1),
    }


def _register_onnx_ops():
    from ..ops.registry import has, op
    if has("onnx.Less"):
        return
    for name, (fn, n_out) in _onnx_ops().items():
        op("onnx." + name, n_out=n_out, group="onnx_import")(fn)


def _generic(opname):
    def f(sd, ctx, n, x):
        fn, n_out = _GENERIC[opname]
        k = len([o for o in n["outputs"]]) if n_out == -1 else n_out
        attrs = {a: (list(v) if isinstance(v, (list, tuple)) else v) for a, v in n["attrs"].items() if not isinstance(v, (torch.Tensor, dict))}
        tens = {a: v for a, v in n["attrs"].items() if isinstance(v, torch.Tensor)}
        ins = list(x)
        while ins and ins[-1] is None:
            ins.pop()
        if opname == "Split":
            attrs["num_outputs"] = k
        if tens:                                     # tensor-valued attributes (ConstantOfShape.value) become constants of the graph
            for a, t in tens.items():
                attrs[a] = t
        return sd._op("onnx." + opname, ins, n_out=k, **attrs)
    return f


_GENERIC = _onnx_ops()

for _name in _GENERIC:
    OP_MAPPERS.setdefault(_name, _generic(_name))


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
        _register_onnx_ops()
        if isinstance(path_or_bytes, (bytes, bytearray, memoryview)):
            data = path_or_bytes
        else:
            with open(path_or_bytes, "rb") as f:
                data = f.read()
        model = parse_model(data)
        sd = self._build(model)
        sd.metadata["onnx.outputs"] = ",".join(model["outputs"])
        sd.metadata["onnx.opset"] = str(model["opset"])
        self.outputs = model["outputs"]
        return sd

    def _build(self, model):
        """A SameDiff for one graph (the model's main graph, or the body of an If / Loop node)."""
        _register_helpers()
        _register_onnx_ops()
        _register_control_flow()
        unsupported = sorted({n["op"] for n in model["nodes"] if n["op"] not in OP_MAPPERS})
        if unsupported:
            raise NotImplementedError(f"ONNX import: no mapping rule for op types {unsupported}")
        sd = SameDiff.create()
        vars_, ctx = {}, {"consts": dict(model["initializers"])}

        def lookup(name):
            if name not in vars_ and name in ctx["consts"]:
                vars_[name] = sd.constant(name, ctx["consts"][name].clone())
            return vars_[name]
        ctx["lookup"] = lookup
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
            for i in n["inputs"]:                       # an initializer that some rule consumed at import time and another reads as data
                if i and i not in vars_ and i in ctx["consts"] and n["op"] in _GENERIC:
                    vars_[i] = sd.constant(i, ctx["consts"][i].clone())
            ins = [vars_.get(i) if i else None for i in n["inputs"]]
            out = OP_MAPPERS[n["op"]](sd, ctx, n, ins)
            outs = out if isinstance(out, (list, tuple)) else [out]
            for name, v in zip(n["outputs"], outs):
                if name and v.name != name:
                    v = sd.renameVariable(v.name, name) or sd.getVariable(name)
                vars_[name] = sd.getVariable(name) if sd.hasVariable(name) else v
        for o in model["outputs"]:                  # a graph output that is a plain input or initializer (Loop bodies pass values through)
            if o not in vars_ or not sd.hasVariable(o):
                if o in ctx["consts"]:
                    lookup(o)
        return sd


def importOnnx(path_or_bytes, trainable=True):
    return OnnxFrameworkImporter(trainable).runImport(path_or_bytes)
