"""Positional op arguments (iArgs / tArgs / bArgs / dArgs, plus the legacy ops' ``dimensions`` and ``scalar``) <-> the
keyword arguments the registry implementations take.

The reference stores the arguments of a graph node positionally: ``FlatNode.extraInteger`` (iArgs), ``extraParams``
(tArgs), ``extraBools`` (bArgs), ``extraTypes`` (dArgs), ``dimensions`` and ``scalar``
(``nd4j-api/.../autodiff/samediff/serde/FlatBuffersMapper.java:735-1005``), in the order each declarable op reads them with
``INT_ARG(i)`` / ``T_ARG(i)`` / ``B_ARG(i)`` (``libnd4j/include/ops/declarable/generic/**``, ``graph/Context.h``).  A node
written by the reference can only be executed here once those positions are turned back into names; ``kwargs_for`` does that
for the ops listed in ``SCHEMAS`` and falls back to a generic rule for the legacy families (reductions take ``dimensions`` +
``keepDims``; scalar ops take the scalar as second operand).
"""
from __future__ import annotations

import torch

INT_MAX = 2147483647


def _names(*names, bools=()):
    """iArgs by position -> keyword names; ``bools``: names whose integer value is a flag."""
    def f(i, t, b, extra):
        kw = {}
        for n, v in zip(names, i):
            if n is None:
                continue
            kw[n] = bool(v) if n in bools else int(v)
        return kw
    return f


def _conv2d(i, t, b, extra):
    kw = dict(zip(("kH", "kW", "sH", "sW", "pH", "pW", "dH", "dW"), (int(v) for v in i[:8])))
    if len(i) > 8:
        kw["isSameMode"] = int(i[8]) == 1
        if int(i[8]) == 2:
            kw["paddingMode"] = "CAUSAL"
    if len(i) > 9:
        kw["dataFormat"] = int(i[9])            # 0 NCHW, 1 NHWC
    if len(i) > 10:
        kw["wFormat"] = int(i[10])        # 0 [kH,kW,iC,oC], 1 [oC,iC,kH,kW], 2 [oC,kH,kW,iC]
    return kw


def _pool2d(i, t, b, extra):
    kw = dict(zip(("kH", "kW", "sH", "sW", "pH", "pW", "dH", "dW"), (int(v) for v in i[:8])))
    if len(i) > 8:
        kw["isSameMode"] = bool(i[8])
    if len(i) > 9:
        kw["extraParam0"] = int(i[9])
    if len(i) > 10:
        kw["dataFormat"] = int(i[10])
    return kw


def _pool3d(i, t, b, extra):
    kw = dict(zip(("kD", "kH", "kW", "sD", "sH", "sW", "pD", "pH", "pW", "dD", "dH", "dW"), (int(v) for v in i[:12])))
    if len(i) > 12:
        kw["isSameMode"] = bool(i[12])
    if len(i) > 13:
        kw["extraParam0"] = int(i[13])
    if len(i) > 14:
        kw["dataFormat"] = int(i[14])           # 0 NCDHW, 1 NDHWC
    return kw


def _reduce(i, t, b, extra):
    dims = extra.get("dimensions")
    dims = [int(d) for d in (dims if dims else i)]
    kw = {}
    if dims and not (len(dims) == 1 and dims[0] == INT_MAX):
        kw["dimensions"] = dims
    if len(b):
        kw["keepDims"] = bool(b[0])
    elif len(t):
        kw["keepDims"] = bool(t[0])
    return kw


def _mmul(i, t, b, extra):
    kw = {}
    for n, v in zip(("transposeX", "transposeY", "transposeZ"), i):
        kw[n] = bool(v)
    if len(t) > 0:
        kw["alpha"] = float(t[0])
    if len(t) > 1:
        kw["beta"] = float(t[1])
    return kw


def _softmax(i, t, b, extra):
    return {"dimension": int(i[0])} if len(i) else {}


def _onehot(i, t, b, extra):
    kw = {}
    if len(i) > 0:
        kw["axis"] = int(i[0])
    if len(i) > 1:
        kw["depth"] = int(i[1])
    if len(t) > 0:
        kw["on"] = float(t[0])
    if len(t) > 1:
        kw["off"] = float(t[1])
    return kw


def _strided_slice(i, t, b, extra):
    kw = dict(zip(("begin_mask", "ellipsis_mask", "end_mask", "new_axis_mask", "shrink_axis_mask"), (int(v) for v in i[:5])))
    rest = [int(v) for v in i[5:]]
    if rest:                                    # begin / end / strides follow when they are static
        n = len(rest) // 3
        kw["begin"], kw["end"], kw["strides"] = rest[:n], rest[n:2 * n], rest[2 * n:3 * n]
    return kw


def _cast(i, t, b, extra):
    from ..nd.dtype import DataType
    if len(i):
        return {"dtype": DataType(int(i[0]))}
    d = extra.get("dtypes") or []
    return {"dtype": DataType(int(d[0]))} if d else {}


def _batchnorm(i, t, b, extra):
    kw = {}
    if len(i) > 0:
        kw["applyScale"] = bool(i[0])
    if len(i) > 1:
        kw["applyOffset"] = bool(i[1])
    if len(i) > 2:
        kw["axis"] = tuple(int(v) for v in i[2:])
    if len(t) > 0:
        kw["epsilon"] = float(t[0])
    return kw


def _linspace(i, t, b, extra):
    kw = {}
    if len(t) > 0:
        kw["start"] = float(t[0])
    if len(t) > 1:
        kw["stop"] = float(t[1])
    if len(t) > 2:
        kw["number"] = int(t[2])
    elif len(i) > 0:
        kw["number"] = int(i[0])
    return kw


def _relu(i, t, b, extra):
    s = extra.get("scalar")
    if s is not None:
        return {"cutoff": float(s.reshape(-1)[0])}
    return {"cutoff": float(t[0])} if len(t) else {}


def _lrelu(i, t, b, extra):
    s = extra.get("scalar")
    if s is not None:
        return {"alpha": float(s.reshape(-1)[0])}
    return {"alpha": float(t[0])} if len(t) else {}


SCHEMAS = {
    "conv2d": _conv2d, "conv2d_bp": _conv2d, "deconv2d": _conv2d, "depthwise_conv2d": _conv2d, "sconv2d": _conv2d,
    "maxpool2d": _pool2d, "avgpool2d": _pool2d, "pnormpool2d": _pool2d,
    "maxpool3dnew": _pool3d, "avgpool3dnew": _pool3d,
    "concat": _names("concatDimension"), "stack": _names("dimension"), "parallel_stack": _names("dimension"),
    "unstack": _names("dimension", "num"), "expand_dims": _names("axis"), "gather": _names("axis"),
    "squeeze": lambda i, t, b, e: ({"dimensions": [int(v) for v in i]} if len(i) else {}),
    "transpose": lambda i, t, b, e: ({"dimensions": [int(v) for v in i]} if len(i) else {}),
    "permute": lambda i, t, b, e: ({"dimensions": [int(v) for v in i]} if len(i) else {}),
    "reshape": lambda i, t, b, e: ({"shape": [int(v) for v in i if int(v) not in (99, 102, -99, -102)]} if len(i) else {}),
    "tile": lambda i, t, b, e: ({"reps": [int(v) for v in i]} if len(i) else {}),
    "mmul": _mmul, "matmul": _mmul,
    "softmax": _softmax, "log_softmax": _softmax,
    "pad": lambda i, t, b, e: dict(({"mode": int(i[0])} if len(i) else {}), **({"padValue": float(t[0])} if len(t) else {})),
    "onehot": _onehot, "strided_slice": _strided_slice, "stridedslice": _strided_slice, "cast": _cast,
    "batchnorm": _batchnorm, "linspace": _linspace, "lin_space": _linspace,
    "relu": _relu, "lrelu": _lrelu, "leakyrelu": _lrelu,
    "argmax": _reduce, "argmin": _reduce, "argamax": _reduce, "argamin": _reduce,
    "cumsum": lambda i, t, b, e: dict(zip(("exclusive", "reverse"), (bool(v) for v in i[:2])), **({"dimensions": [int(v) for v in i[2:]]} if len(i) > 2 else {})),
    "reverse": lambda i, t, b, e: ({"dimensions": [int(v) for v in i]} if len(i) else {}),
    "dropout": lambda i, t, b, e: dict(({"seed": int(i[0])} if len(i) else {}), **({"p": float(t[0])} if len(t) else {})),
    "layer_norm": lambda i, t, b, e: dict(({"dimensions": [int(v) for v in i]} if len(i) else {}), **({"channelsFirst": bool(b[0])} if len(b) else {})),
    "clipbyvalue": lambda i, t, b, e: ({"clipValueMin": float(t[0]), "clipValueMax": float(t[1])} if len(t) > 1 else {}),
    "clipbynorm": lambda i, t, b, e: dict(({"clipValue": float(t[0])} if len(t) else {}), **({"dimensions": [int(v) for v in i]} if len(i) else {})),
    "tensorarrayv3": lambda i, t, b, e: {}, "tensorarraywritev3": lambda i, t, b, e: {}, "tensorarrayreadv3": lambda i, t, b, e: {},
    "enter": lambda i, t, b, e: {}, "range": lambda i, t, b, e: {},
}

_REDUCE_FAMILIES = ("REDUCE_FLOAT", "REDUCE_SAME", "REDUCE_LONG", "REDUCE_BOOL", "INDEX_REDUCE", "SUMMARYSTATS", "REDUCE_3")
_SCALAR_FAMILIES = ("SCALAR", "SCALAR_BOOL")


def kwargs_for(op_name, op_type, iargs=(), targs=(), bargs=(), dimensions=None, scalar=None, dtypes=None):
    """Keyword arguments for the registry op ``op_name`` from a node's positional arguments.  ``op_type`` is the schema's OpType
    name (``"CUSTOM"``, ``"REDUCE_SAME"``, ...)."""
    def _l(v):
        return [] if v is None else list(v)
    i, t, b = _l(iargs), _l(targs), _l(bargs)
    extra = {"dimensions": list(dimensions) if dimensions is not None and len(dimensions) else None, "scalar": scalar,
             "dtypes": _l(dtypes)}
    f = SCHEMAS.get(op_name)
    if f is not None:
        return f(i, t, b, extra)
    if op_type in _REDUCE_FAMILIES or op_name.startswith("reduce_"):
        return _reduce(i, t, b, extra)
    return {}


def scalar_operand(op_type, scalar, like=None):
    """Legacy scalar ops carry their second operand in ``FlatNode.scalar``."""
    if op_type in _SCALAR_FAMILIES and scalar is not None:
        return scalar if isinstance(scalar, torch.Tensor) else torch.as_tensor(scalar)
    return None
