"""TensorFlow frozen-graph (``GraphDef`` protobuf) -> SameDiff import (``nd4j/samediff-import/samediff-import-tensorflow``,
``TFGraphMapper``).  Parsed with the bundled protobuf wire reader (TensorFlow itself is not needed).  ``Const`` nodes
become constants (or variables with ``trainable=True``), ``Placeholder`` nodes placeholders; data layout stays NHWC
as in the source graph (helper ops ``tf_conv2d`` / ``tf_pool`` do the layout changes around the NCHW kernels)."""
from __future__ import annotations

import numpy as np
import torch

from ..nd.dtype import DataType
from ..samediff.core import SameDiff
from . import protowire as pw

_TF_DTYPES = {1: np.float32, 2: np.float64, 3: np.int32, 4: np.uint8, 5: np.int16, 6: np.int8, 9: np.int64, 10: np.bool_, 19: np.float16}
_TF_TO_DT = {1: DataType.FLOAT, 2: DataType.DOUBLE, 3: DataType.INT, 9: DataType.LONG, 10: DataType.BOOL, 19: DataType.HALF, 14: DataType.BFLOAT16}


def _shape(buf):
    s = pw.decode(buf)
    if 3 in s and s[3][0]:
        return None
    return [pw.signed(pw.decode(d).get(1, [0])[0]) for d in s.get(2, [])]


def _tensor(buf):
    t = pw.decode(buf)
    dt = t.get(1, [1])[0]
    shape = _shape(t[2][0]) if 2 in t else []
    npdt = _TF_DTYPES.get(dt, np.float32)
    n = int(np.prod(shape)) if shape else 1
    if 4 in t and len(t[4][0]):
        arr = np.frombuffer(bytes(t[4][0]), dtype=np.dtype(npdt).newbyteorder("<"))
    elif 5 in t:
        arr = np.asarray(pw.packed_fixed(t[5], "f"), dtype=np.float32)
    elif 6 in t:
        arr = np.asarray(pw.packed_fixed(t[6], "d"), dtype=np.float64)
    elif 7 in t:
        arr = np.asarray(pw.packed_varints(t[7]), dtype=np.int64).astype(npdt)
    elif 10 in t:
        arr = np.asarray(pw.packed_varints(t[10]), dtype=np.int64)
    elif 11 in t:
        arr = np.asarray(pw.packed_varints(t[11]), dtype=np.int64).astype(np.bool_)
    else:
        arr = np.zeros(n, dtype=npdt)
    if arr.size == 1 and n > 1:
        arr = np.full(n, arr.reshape(-1)[0], dtype=arr.dtype)      # scalar splat encoding
    return torch.from_numpy(np.array(arr).reshape(shape or ()))


def _attr(buf):
    a = pw.decode(buf)
    if 2 in a: return bytes(a[2][0]).decode("utf-8", "replace")
    if 3 in a: return pw.signed(a[3][0])
    if 4 in a: return pw.packed_fixed(a[4], "f")[0]
    if 5 in a: return bool(a[5][0])
    if 6 in a: return ("dtype", a[6][0])
    if 7 in a: return ("shape", _shape(a[7][0]))
    if 8 in a: return _tensor(a[8][0])
    if 1 in a:
        l = pw.decode(a[1][0])
        if 3 in l: return pw.packed_varints(l[3])
        if 4 in l: return pw.packed_fixed(l[4], "f")
        if 2 in l: return [bytes(s).decode() for s in l[2]]
        return []
    return None


def parse_graphdef(data):
    g = pw.decode(data)
    nodes = []
    for nb in g.get(1, []):
        n = pw.decode(nb)
        attrs = {}
        for e in n.get(5, []):
            kv = pw.decode(e)
            attrs[pw.string(kv[1][0])] = _attr(kv[2][0]) if 2 in kv else None
        nodes.append({"name": pw.string(n[1][0]), "op": pw.string(n[2][0]), "inputs": [pw.string(s) for s in n.get(3, [])], "attrs": attrs})
    return nodes


def _register_helpers():
    import torch.nn.functional as F
    from ..ops.registry import has, op
    if has("tf_conv2d"):
        return

    def _same_pad(x, k, s, d):
        pads = []
        for i in (1, 0):
            size = x.shape[2 + i]
            out = -(-size // s[i])
            tot = max((out - 1) * s[i] + (k[i] - 1) * d[i] + 1 - size, 0)
            pads += [tot // 2, tot - tot // 2]
        return F.pad(x, pads) if any(pads) else x

    @op("tf_conv2d")
    def tf_conv2d(x, w, strides=(1, 1, 1, 1), padding="SAME", dilations=(1, 1, 1, 1), data_format="NHWC", depthwise=False, **kw):
        nhwc = data_format == "NHWC"
        if nhwc:
            x = x.permute(0, 3, 1, 2)
        s = (strides[1], strides[2]) if nhwc else (strides[2], strides[3])
        d = (dilations[1], dilations[2]) if nhwc else (dilations[2], dilations[3])
        groups = 1
        if depthwise:                                   # [kh, kw, in, mult] -> [in*mult, 1, kh, kw]
            kh, kw_, cin, mult = w.shape
            wt = w.permute(2, 3, 0, 1).reshape(cin * mult, 1, kh, kw_)
            groups = cin
        else:
            wt = w.permute(3, 2, 0, 1)                  # HWIO -> OIHW
        if padding == "SAME":
            x = _same_pad(x, wt.shape[2:], s, d)
        y = F.conv2d(x, wt.to(x.dtype), None, s, 0, d, groups)
        return y.permute(0, 2, 3, 1) if nhwc else y

    @op("tf_pool")
    def tf_pool(x, kind="max", ksize=(1, 2, 2, 1), strides=(1, 2, 2, 1), padding="VALID", data_format="NHWC", **kw):
        nhwc = data_format == "NHWC"
        if nhwc:
            x = x.permute(0, 3, 1, 2)
        k = (ksize[1], ksize[2]) if nhwc else (ksize[2], ksize[3])
        s = (strides[1], strides[2]) if nhwc else (strides[2], strides[3])
        if padding == "SAME":
            if kind == "max":
                pads = []
                for i in (1, 0):
                    size = x.shape[2 + i]
                    tot = max((-(-size // s[i]) - 1) * s[i] + k[i] - size, 0)
                    pads += [tot // 2, tot - tot // 2]
                x = F.pad(x, pads, value=float("-inf"))
                y = F.max_pool2d(x, k, s)
            else:
                ones = _same_pad(torch.ones_like(x), k, s, (1, 1))
                y = F.avg_pool2d(_same_pad(x, k, s, (1, 1)), k, s) / F.avg_pool2d(ones, k, s).clamp(min=1e-12)
        else:
            y = F.max_pool2d(x, k, s) if kind == "max" else F.avg_pool2d(x, k, s)
        return y.permute(0, 2, 3, 1) if nhwc else y

    @op("tf_bias_add")
    def tf_bias_add(x, b, data_format="NHWC", **kw):
        if data_format == "NCHW" and x.dim() > 2:
            return x + b.reshape([1, -1] + [1] * (x.dim() - 2))
        return x + b

    @op("tf_fused_batchnorm", n_out=1)
    def tf_fused_batchnorm(x, scale, offset, mean, var, epsilon=1e-3, data_format="NHWC", **kw):
        shp = [1, 1, 1, -1] if data_format == "NHWC" else [1, -1, 1, 1]
        return (x - mean.reshape(shp)) * (scale.reshape(shp) * torch.rsqrt(var.reshape(shp) + epsilon)) + offset.reshape(shp)


def _base(name):
    name = name[1:] if name.startswith("^") else name
    return name.split(":")[0], int(name.split(":")[1]) if ":" in name else 0


class TensorflowFrameworkImporter:
    UNARY = {"Relu": "relu", "Relu6": "relu6", "Sigmoid": "sigmoid", "Tanh": "tanh", "Exp": "exp", "Log": "log", "Sqrt": "sqrt", "Rsqrt": "rsqrt",
             "Neg": "neg", "Abs": "abs", "Identity": "identity", "StopGradient": "identity", "Softplus": "softplus", "Erf": "erf", "Square": "square",
             "Floor": "floor", "Elu": "elu", "Selu": "selu"}
    BINARY = {"Add": "add", "AddV2": "add", "Sub": "subtract", "Mul": "multiply", "RealDiv": "divide", "Div": "divide", "Maximum": "maximum",
              "Minimum": "minimum", "Pow": "Pow", "SquaredDifference": "squaredsubtract"}
    REDUCE = {"Mean": "reduce_mean", "Sum": "reduce_sum", "Max": "reduce_max", "Min": "reduce_min", "Prod": "reduce_prod"}

    def __init__(self, trainable=False):
        self.trainable = trainable

    def runImport(self, path_or_bytes, dynamicVariables=None):
        _register_helpers()
        if isinstance(path_or_bytes, (bytes, bytearray, memoryview)):
            data = path_or_bytes
        else:
            with open(path_or_bytes, "rb") as f:
                data = f.read()
        nodes = parse_graphdef(data)
        known = set(self.UNARY) | set(self.BINARY) | set(self.REDUCE) | {"Const", "Placeholder", "PlaceholderWithDefault", "MatMul", "BiasAdd", "Conv2D", "DepthwiseConv2dNative", "MaxPool", "AvgPool", "Reshape", "Softmax",
                                                                           "LogSoftmax", "Squeeze", "ExpandDims", "ConcatV2", "Transpose", "FusedBatchNorm", "FusedBatchNormV3", "Pad", "Cast",
                                                                           "LeakyRelu", "NoOp", "Shape", "Pack", "StridedSlice", "GatherV2", "ArgMax"}
        unsupported = sorted({n["op"] for n in nodes if n["op"] not in known})
        if unsupported:
            raise NotImplementedError(f"TensorFlow import: no mapping rule for op types {unsupported}")
        sd = SameDiff.create()
        vars_, consts = {}, {}

        def inp(n, i):
            nm, idx = _base(n["inputs"][i])
            return vars_[nm]

        def cval(n, i):
            nm, _ = _base(n["inputs"][i])
            if nm not in consts:
                raise ValueError(f"TensorFlow import: input {i} of {n['name']} ({n['op']}) must be a constant")
            return consts[nm]
        for n in nodes:
            op_, a, name = n["op"], n["attrs"], n["name"]
            data_in = [i for i in n["inputs"] if not i.startswith("^")]
            n = dict(n, inputs=data_in)
            if op_ == "NoOp":
                continue
            if op_ == "Const":
                t = a["value"]
                consts[name] = t
                vars_[name] = sd.var(name, t.clone()) if (self.trainable and t.is_floating_point() and t.dim() >= 1) else sd.constant(name, t.clone())
            elif op_ in ("Placeholder", "PlaceholderWithDefault"):
                dt = _TF_TO_DT.get(a.get("dtype", ("dtype", 1))[1], DataType.FLOAT)
                shp = a.get("shape", ("shape", None))[1]
                vars_[name] = sd.placeHolder(name, dt, *(shp or []))
            elif op_ in self.UNARY:
                vars_[name] = sd._op(self.UNARY[op_], [inp(n, 0)], name=name)
            elif op_ in self.BINARY:
                vars_[name] = sd._op(self.BINARY[op_], [inp(n, 0), inp(n, 1)], name=name)
            elif op_ in self.REDUCE:
                ax = cval(n, 1).reshape(-1).tolist()
                vars_[name] = sd._op(self.REDUCE[op_], [inp(n, 0)], name=name, dimensions=[int(v) for v in ax], keepDims=bool(a.get("keep_dims", False)))
            elif op_ == "MatMul":
                vars_[name] = sd._op("matmul", [inp(n, 0), inp(n, 1)], name=name, transposeX=bool(a.get("transpose_a", False)), transposeY=bool(a.get("transpose_b", False)))
            elif op_ == "BiasAdd":
                vars_[name] = sd._op("tf_bias_add", [inp(n, 0), inp(n, 1)], name=name, data_format=a.get("data_format", "NHWC"))
            elif op_ in ("Conv2D", "DepthwiseConv2dNative"):
                vars_[name] = sd._op("tf_conv2d", [inp(n, 0), inp(n, 1)], name=name, strides=list(a.get("strides", [1, 1, 1, 1])), padding=a.get("padding", "SAME"),
                                     dilations=list(a.get("dilations", [1, 1, 1, 1])), data_format=a.get("data_format", "NHWC"), depthwise=op_ != "Conv2D")
            elif op_ in ("MaxPool", "AvgPool"):
                vars_[name] = sd._op("tf_pool", [inp(n, 0)], name=name, kind="max" if op_ == "MaxPool" else "avg", ksize=list(a["ksize"]), strides=list(a["strides"]),
                                     padding=a.get("padding", "VALID"), data_format=a.get("data_format", "NHWC"))
            elif op_ == "Reshape":
                vars_[name] = sd._op("reshape", [inp(n, 0)], name=name, shape=[int(v) for v in cval(n, 1).reshape(-1).tolist()])
            elif op_ in ("Softmax", "LogSoftmax"):
                vars_[name] = sd._op("softmax" if op_ == "Softmax" else "log_softmax", [inp(n, 0)], name=name, dimension=-1)
            elif op_ == "Squeeze":
                dims = a.get("squeeze_dims") or None
                vars_[name] = sd._op("squeeze", [inp(n, 0)], name=name, dimensions=None if not dims else [int(v) for v in dims])
            elif op_ == "ExpandDims":
                vars_[name] = sd._op("expand_dims", [inp(n, 0)], name=name, axis=int(cval(n, 1)))
            elif op_ == "ConcatV2":
                vars_[name] = sd._op("concat", [inp(n, i) for i in range(len(n["inputs"]) - 1)], name=name, concatDimension=int(cval(n, len(n["inputs"]) - 1)))
            elif op_ == "Pack":
                vars_[name] = sd._op("stack", [inp(n, i) for i in range(len(n["inputs"]))], name=name, axis=int(a.get("axis", 0)))
            elif op_ == "Transpose":
                vars_[name] = sd._op("permute", [inp(n, 0)], name=name, dimensions=[int(v) for v in cval(n, 1).tolist()])
            elif op_ in ("FusedBatchNorm", "FusedBatchNormV3"):
                vars_[name] = sd._op("tf_fused_batchnorm", [inp(n, i) for i in range(5)], name=name, epsilon=float(a.get("epsilon", 1e-3)), data_format=a.get("data_format", "NHWC"))
            elif op_ == "Pad":
                vars_[name] = sd._op("pad", [inp(n, 0)], name=name, paddings=cval(n, 1).tolist(), mode="CONSTANT", constant=0.0)
            elif op_ == "Cast":
                vars_[name] = sd._op("cast", [inp(n, 0)], name=name, dtype=int(_TF_TO_DT.get(a["DstT"][1], DataType.FLOAT)))
            elif op_ == "LeakyRelu":
                vars_[name] = sd._op("leakyrelu", [inp(n, 0)], name=name, alpha=float(a.get("alpha", 0.2)))
            elif op_ == "Shape":
                vars_[name] = sd._op("shape_of", [inp(n, 0)], name=name)
            elif op_ == "GatherV2":
                vars_[name] = sd._op("gather", [inp(n, 0), inp(n, 1)], name=name, axis=int(cval(n, 2)))
            elif op_ == "ArgMax":
                vars_[name] = sd._op("argmax", [inp(n, 0)], name=name, dimensions=[int(cval(n, 1))])
            elif op_ == "StridedSlice":
                b, e, s = (cval(n, i).reshape(-1).tolist() for i in (1, 2, 3))
                vars_[name] = sd._op("strided_slice", [inp(n, 0)], name=name, begin=[int(v) for v in b], end=[int(v) for v in e], strides=[int(v) for v in s],
                                     beginMask=int(a.get("begin_mask", 0)), endMask=int(a.get("end_mask", 0)), ellipsisMask=int(a.get("ellipsis_mask", 0)),
                                     newAxisMask=int(a.get("new_axis_mask", 0)), shrinkAxisMask=int(a.get("shrink_axis_mask", 0)))
        consumed = {_base(i)[0] for n in nodes for i in n["inputs"]}
        self.outputs = [n["name"] for n in nodes if n["name"] not in consumed and n["op"] not in ("Const", "Placeholder", "NoOp")]
        return sd


def importFrozenTF(path_or_bytes, trainable=False):
    return TensorflowFrameworkImporter(trainable).runImport(path_or_bytes)
