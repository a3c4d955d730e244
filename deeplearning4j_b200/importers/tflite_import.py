"""TensorFlow Lite flatbuffer models -> SameDiff (the model format behind ``nd4j-tensorflow-lite`` ``TensorFlowLiteRunner``, which
hands the file to the vendor interpreter; here the graph is imported and runs on this framework's kernels).

The file is a FlatBuffers ``Model`` (identifier ``TFL3``): operator codes, sub-graphs of tensors + operators, and the constant
buffers.  The tables below restate the parts of the public TFLite schema (version 3) that float models use; every operator
becomes one ``tflite.<NAME>`` registry op that implements the TFLite semantics on tensors (NHWC activations, ``[O, KH, KW, I]``
filters, TensorFlow SAME padding, fused activation functions), so an imported graph serialises and differentiates like any other.
Constant tensors that are stored quantised (int8 / uint8 / int16 with scale and zero point, per tensor or per axis) or as fp16
are dequantised at import; graphs whose *activations* are quantised are refused.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from ..nd.dtype import DataType
from ..samediff.core import SameDiff
from ..samediff.serde.flatbuffers import decode, table, union, vec

# ----------------------------------------------------------------------------- schema
_OPTIONS = {
    1: "Conv2DOptions", 2: "DepthwiseConv2DOptions", 5: "Pool2DOptions", 8: "FullyConnectedOptions", 9: "SoftmaxOptions",
    10: "ConcatenationOptions", 11: "AddOptions", 12: "L2NormOptions", 15: "ResizeBilinearOptions", 17: "ReshapeOptions",
    19: "SpaceToDepthOptions", 21: "MulOptions", 23: "GatherOptions", 27: "ReducerOptions", 28: "SubOptions", 29: "DivOptions",
    30: "SqueezeOptions", 32: "StridedSliceOptions", 35: "SplitOptions", 37: "CastOptions", 40: "ArgMaxOptions",
    47: "TransposeConvOptions", 55: "ArgMinOptions", 57: "PackOptions", 59: "OneHotOptions", 62: "UnpackOptions",
    72: "ResizeNearestNeighborOptions", 73: "LeakyReluOptions", 75: "MirrorPadOptions", 77: "SplitVOptions",
    92: "DepthToSpaceOptions", 99: "BatchMatMulOptions", 100: "CumsumOptions", 114: "GeluOptions",
}
OPTION_IDS = {v: k for k, v in _OPTIONS.items()}

TFL_SCHEMA = {
    "QuantizationParameters": [("min", vec("float")), ("max", vec("float")), ("scale", vec("float")), ("zero_point", vec("long")),
                               ("details_type", "ubyte"), ("details", "uint"), ("quantized_dimension", "int")],
    "Tensor": [("shape", vec("int")), ("type", "byte"), ("buffer", "uint"), ("name", "string"),
               ("quantization", table("QuantizationParameters")), ("is_variable", "bool"), ("sparsity", "uint"),
               ("shape_signature", vec("int"))],
    "OperatorCode": [("deprecated_builtin_code", "byte"), ("custom_code", "string"), ("version", "int", 1), ("builtin_code", "int")],
    "Operator": [("opcode_index", "uint"), ("inputs", vec("int")), ("outputs", vec("int")), ("builtin_options_type", "ubyte"),
                 ("builtin_options", union("builtin_options_type", _OPTIONS)), ("custom_options", vec("ubyte")),
                 ("custom_options_format", "byte"), ("mutating_variable_inputs", vec("bool")), ("intermediates", vec("int"))],
    "SubGraph": [("tensors", vec(table("Tensor"))), ("inputs", vec("int")), ("outputs", vec("int")),
                 ("operators", vec(table("Operator"))), ("name", "string")],
    "Buffer": [("data", vec("ubyte")), ("offset", "ulong"), ("size", "ulong")],
    "Model": [("version", "uint"), ("operator_codes", vec(table("OperatorCode"))), ("subgraphs", vec(table("SubGraph"))),
              ("description", "string"), ("buffers", vec(table("Buffer")))],
    # builtin option tables
    "Conv2DOptions": [("padding", "byte"), ("stride_w", "int"), ("stride_h", "int"), ("fused_activation_function", "byte"),
                      ("dilation_w_factor", "int", 1), ("dilation_h_factor", "int", 1)],
    "DepthwiseConv2DOptions": [("padding", "byte"), ("stride_w", "int"), ("stride_h", "int"), ("depth_multiplier", "int"),
                               ("fused_activation_function", "byte"), ("dilation_w_factor", "int", 1), ("dilation_h_factor", "int", 1)],
    "Pool2DOptions": [("padding", "byte"), ("stride_w", "int"), ("stride_h", "int"), ("filter_width", "int"), ("filter_height", "int"),
                      ("fused_activation_function", "byte")],
    "FullyConnectedOptions": [("fused_activation_function", "byte"), ("weights_format", "byte"), ("keep_num_dims", "bool"),
                              ("asymmetric_quantize_inputs", "bool")],
    "SoftmaxOptions": [("beta", "float")],
    "ConcatenationOptions": [("axis", "int"), ("fused_activation_function", "byte")],
    "AddOptions": [("fused_activation_function", "byte"), ("pot_scale_int16", "bool", True)],
    "SubOptions": [("fused_activation_function", "byte"), ("pot_scale_int16", "bool", True)],
    "MulOptions": [("fused_activation_function", "byte")],
    "DivOptions": [("fused_activation_function", "byte")],
    "L2NormOptions": [("fused_activation_function", "byte")],
    "ResizeBilinearOptions": [("new_height", "int"), ("new_width", "int"), ("align_corners", "bool"), ("half_pixel_centers", "bool")],
    "ResizeNearestNeighborOptions": [("align_corners", "bool"), ("half_pixel_centers", "bool")],
    "ReshapeOptions": [("new_shape", vec("int"))],
    "SpaceToDepthOptions": [("block_size", "int")],
    "DepthToSpaceOptions": [("block_size", "int")],
    "GatherOptions": [("axis", "int"), ("batch_dims", "int")],
    "ReducerOptions": [("keep_dims", "bool")],
    "SqueezeOptions": [("squeeze_dims", vec("int"))],
    "StridedSliceOptions": [("begin_mask", "int"), ("end_mask", "int"), ("ellipsis_mask", "int"), ("new_axis_mask", "int"),
                            ("shrink_axis_mask", "int"), ("offset", "bool")],
    "SplitOptions": [("num_splits", "int")],
    "SplitVOptions": [("num_splits", "int")],
    "CastOptions": [("in_data_type", "byte"), ("out_data_type", "byte")],
    "ArgMaxOptions": [("output_type", "byte")],
    "ArgMinOptions": [("output_type", "byte")],
    "TransposeConvOptions": [("padding", "byte"), ("stride_w", "int"), ("stride_h", "int"), ("fused_activation_function", "byte")],
    "PackOptions": [("values_count", "int"), ("axis", "int")],
    "UnpackOptions": [("num", "int"), ("axis", "int")],
    "OneHotOptions": [("axis", "int")],
    "LeakyReluOptions": [("alpha", "float")],
    "MirrorPadOptions": [("mode", "byte")],
    "BatchMatMulOptions": [("adj_x", "bool"), ("adj_y", "bool"), ("asymmetric_quantize_inputs", "bool")],
    "CumsumOptions": [("exclusive", "bool"), ("reverse", "bool")],
    "GeluOptions": [("approximate", "bool")],
}

BUILTIN = {
    0: "ADD", 1: "AVERAGE_POOL_2D", 2: "CONCATENATION", 3: "CONV_2D", 4: "DEPTHWISE_CONV_2D", 5: "DEPTH_TO_SPACE", 6: "DEQUANTIZE",
    7: "EMBEDDING_LOOKUP", 8: "FLOOR", 9: "FULLY_CONNECTED", 11: "L2_NORMALIZATION", 14: "LOGISTIC", 17: "MAX_POOL_2D", 18: "MUL",
    19: "RELU", 20: "RELU_N1_TO_1", 21: "RELU6", 22: "RESHAPE", 23: "RESIZE_BILINEAR", 25: "SOFTMAX", 26: "SPACE_TO_DEPTH", 28: "TANH",
    34: "PAD", 36: "GATHER", 39: "TRANSPOSE", 40: "MEAN", 41: "SUB", 42: "DIV", 43: "SQUEEZE", 45: "STRIDED_SLICE", 47: "EXP",
    49: "SPLIT", 50: "LOG_SOFTMAX", 53: "CAST", 54: "PRELU", 55: "MAXIMUM", 56: "ARG_MAX", 57: "MINIMUM", 58: "LESS", 59: "NEG",
    60: "PADV2", 61: "GREATER", 62: "GREATER_EQUAL", 63: "LESS_EQUAL", 64: "SELECT", 65: "SLICE", 66: "SIN", 67: "TRANSPOSE_CONV",
    69: "TILE", 70: "EXPAND_DIMS", 71: "EQUAL", 72: "NOT_EQUAL", 73: "LOG", 74: "SUM", 75: "SQRT", 76: "RSQRT", 77: "SHAPE", 78: "POW",
    79: "ARG_MIN", 81: "REDUCE_PROD", 82: "REDUCE_MAX", 83: "PACK", 84: "LOGICAL_OR", 85: "ONE_HOT", 86: "LOGICAL_AND",
    87: "LOGICAL_NOT", 88: "UNPACK", 89: "REDUCE_MIN", 90: "FLOOR_DIV", 92: "SQUARE", 93: "ZEROS_LIKE", 94: "FILL", 95: "FLOOR_MOD",
    96: "RANGE", 97: "RESIZE_NEAREST_NEIGHBOR", 98: "LEAKY_RELU", 99: "SQUARED_DIFFERENCE", 100: "MIRROR_PAD", 101: "ABS",
    102: "SPLIT_V", 104: "CEIL", 105: "REVERSE_V2", 106: "ADD_N", 107: "GATHER_ND", 108: "COS", 110: "RANK", 111: "ELU",
    116: "ROUND", 117: "HARD_SWISH", 123: "SELECT_V2", 126: "BATCH_MATMUL", 128: "CUMSUM", 150: "GELU",
    12: "L2_POOL_2D", 37: "BATCH_TO_SPACE_ND", 38: "SPACE_TO_BATCH_ND", 48: "TOPK_V2", 68: "SPARSE_TO_DENSE", 91: "REDUCE_ANY",
    109: "WHERE", 113: "MATRIX_DIAG", 115: "MATRIX_SET_DIAG", 122: "SCATTER_ND", 125: "SEGMENT_SUM", 130: "BROADCAST_TO",
    140: "REDUCE_ALL", 145: "BROADCAST_ARGS", 152: "RELU_0_TO_1", 153: "UNSORTED_SEGMENT_PROD", 154: "UNSORTED_SEGMENT_MAX",
    155: "UNSORTED_SEGMENT_SUM", 156: "ATAN2", 157: "UNSORTED_SEGMENT_MIN", 158: "SIGN",
}
BUILTIN_CODES = {v: k for k, v in BUILTIN.items()}

_TENSOR_TYPES = {0: torch.float32, 1: torch.float16, 2: torch.int32, 3: torch.uint8, 4: torch.int64, 6: torch.bool, 7: torch.int16,
                 9: torch.int8, 10: torch.float64}
_DL4J_TYPES = {0: DataType.FLOAT, 1: DataType.HALF, 2: DataType.INT, 3: DataType.UBYTE, 4: DataType.LONG, 6: DataType.BOOL,
               7: DataType.SHORT, 9: DataType.BYTE, 10: DataType.DOUBLE}
TENSOR_TYPE_IDS = {v: k for k, v in _TENSOR_TYPES.items()}


# ----------------------------------------------------------------------------- operator semantics on tensors
def _ints(t):
    return [int(v) for v in (t.reshape(-1).tolist() if isinstance(t, torch.Tensor) else t)]


def _fused(y, code):
    if code == 1: return torch.relu(y)
    if code == 2: return y.clamp(-1.0, 1.0)
    if code == 3: return y.clamp(0.0, 6.0)
    if code == 4: return torch.tanh(y)
    if code == 5: return torch.signbit(y).to(y.dtype)
    return y


def _same_pads(size, k, s, d):
    """TensorFlow SAME: output ceil(size / s); the odd pixel of the total padding goes to the end."""
    eff = (k - 1) * d + 1
    total = max((math.ceil(size / s) - 1) * s + eff - size, 0)
    return total // 2, total - total // 2


def _pad_nchw(x, padding, kh, kw, sh, sw, dh=1, dw=1, value=0.0):
    if padding == 1:                                   # VALID
        return x
    (t, b), (l, r) = _same_pads(x.shape[2], kh, sh, dh), _same_pads(x.shape[3], kw, sw, dw)
    return torch.nn.functional.pad(x, (l, r, t, b), value=value) if (t or b or l or r) else x


def _tflite_ops():
    F = torch.nn.functional
    ops = {}

    def reg(name, n_out=1):
        def d(fn):
            ops[name] = (fn, n_out)
            return fn
        return d

    @reg("CONV_2D")
    def conv2d(x, w, b=None, padding=0, stride_w=1, stride_h=1, fused_activation_function=0, dilation_w_factor=1, dilation_h_factor=1, **kw):
        xn = _pad_nchw(x.permute(0, 3, 1, 2), padding, w.shape[1], w.shape[2], stride_h, stride_w, dilation_h_factor, dilation_w_factor)
        y = F.conv2d(xn, w.permute(0, 3, 1, 2).to(x.dtype), None if b is None else b.to(x.dtype), (stride_h, stride_w), 0,
                     (dilation_h_factor, dilation_w_factor), groups=x.shape[3] // w.shape[3])
        return _fused(y.permute(0, 2, 3, 1), fused_activation_function)

    @reg("DEPTHWISE_CONV_2D")
    def depthwise(x, w, b=None, padding=0, stride_w=1, stride_h=1, depth_multiplier=1, fused_activation_function=0,
                  dilation_w_factor=1, dilation_h_factor=1, **kw):
        xn = _pad_nchw(x.permute(0, 3, 1, 2), padding, w.shape[1], w.shape[2], stride_h, stride_w, dilation_h_factor, dilation_w_factor)
        y = F.conv2d(xn, w.permute(3, 0, 1, 2).to(x.dtype), None if b is None else b.to(x.dtype), (stride_h, stride_w), 0,
                     (dilation_h_factor, dilation_w_factor), groups=x.shape[3])
        return _fused(y.permute(0, 2, 3, 1), fused_activation_function)

    @reg("TRANSPOSE_CONV")
    def transpose_conv(output_shape, w, x, b=None, padding=0, stride_w=1, stride_h=1, fused_activation_function=0, **kw):
        oh, ow = _ints(output_shape)[1:3]
        kh, kw_ = w.shape[1], w.shape[2]
        full = F.conv_transpose2d(x.permute(0, 3, 1, 2), w.permute(3, 0, 1, 2).to(x.dtype), None, (stride_h, stride_w))
        if padding == 0:                               # SAME: crop what the forward convolution would have padded
            t, _ = _same_pads(oh, kh, stride_h, 1)
            l, _ = _same_pads(ow, kw_, stride_w, 1)
        else:
            t = l = 0
        y = full[:, :, t:t + oh, l:l + ow]
        if y.shape[2] < oh or y.shape[3] < ow:
            y = F.pad(y, (0, ow - y.shape[3], 0, oh - y.shape[2]))
        if b is not None:
            y = y + b.to(y.dtype).reshape(1, -1, 1, 1)
        return _fused(y.permute(0, 2, 3, 1), fused_activation_function)

    @reg("MAX_POOL_2D")
    def max_pool(x, padding=0, stride_w=1, stride_h=1, filter_width=1, filter_height=1, fused_activation_function=0, **kw):
        xn = _pad_nchw(x.permute(0, 3, 1, 2), padding, filter_height, filter_width, stride_h, stride_w, value=float("-inf"))
        return _fused(F.max_pool2d(xn, (filter_height, filter_width), (stride_h, stride_w)).permute(0, 2, 3, 1), fused_activation_function)

    @reg("AVERAGE_POOL_2D")
    def avg_pool(x, padding=0, stride_w=1, stride_h=1, filter_width=1, filter_height=1, fused_activation_function=0, **kw):
        xc = x.permute(0, 3, 1, 2)
        xn = _pad_nchw(xc, padding, filter_height, filter_width, stride_h, stride_w)
        k, s = (filter_height, filter_width), (stride_h, stride_w)
        y = F.avg_pool2d(xn, k, s)
        if xn.shape != xc.shape:                       # padded cells do not count towards the mean
            cnt = F.avg_pool2d(_pad_nchw(torch.ones_like(xc[:1, :1]), padding, filter_height, filter_width, stride_h, stride_w), k, s)
            y = y / cnt
        return _fused(y.permute(0, 2, 3, 1), fused_activation_function)

    @reg("FULLY_CONNECTED")
    def fully_connected(x, w, b=None, fused_activation_function=0, weights_format=0, keep_num_dims=False, **kw):
        x2 = x if keep_num_dims else x.reshape(-1, w.shape[1])
        y = x2 @ w.to(x.dtype).t()
        if b is not None:
            y = y + b.to(y.dtype)
        return _fused(y, fused_activation_function)

    @reg("BATCH_MATMUL")
    def batch_matmul(a, b, adj_x=False, adj_y=False, **kw):
        return (a.transpose(-1, -2) if adj_x else a) @ (b.transpose(-1, -2) if adj_y else b)

    def binary(name, fn):
        @reg(name)
        def f(a, b, fused_activation_function=0, **kw):
            return _fused(fn(a, b), fused_activation_function)
    binary("ADD", torch.add); binary("SUB", torch.sub); binary("MUL", torch.mul)
    binary("DIV", lambda a, b: torch.div(a, b) if a.is_floating_point() else torch.div(a, b, rounding_mode="trunc"))
    binary("MAXIMUM", torch.maximum); binary("MINIMUM", torch.minimum); binary("POW", torch.pow)
    binary("SQUARED_DIFFERENCE", lambda a, b: (a - b) ** 2)
    binary("FLOOR_DIV", lambda a, b: torch.div(a, b, rounding_mode="floor"))
    binary("FLOOR_MOD", torch.remainder)
    for nm, fn in (("LESS", torch.lt), ("GREATER", torch.gt), ("GREATER_EQUAL", torch.ge), ("LESS_EQUAL", torch.le), ("EQUAL", torch.eq),
                   ("NOT_EQUAL", torch.ne), ("LOGICAL_OR", torch.logical_or), ("LOGICAL_AND", torch.logical_and)):
        binary(nm, fn)

    def unary(name, fn):
        @reg(name)
        def f(x, **kw):
            return fn(x)
    for nm, fn in (("LOGISTIC", torch.sigmoid), ("TANH", torch.tanh), ("RELU", torch.relu), ("RELU6", lambda x: x.clamp(0, 6)),
                   ("RELU_N1_TO_1", lambda x: x.clamp(-1, 1)), ("EXP", torch.exp), ("LOG", torch.log), ("SQRT", torch.sqrt),
                   ("RSQRT", torch.rsqrt), ("SQUARE", torch.square), ("ABS", torch.abs), ("NEG", torch.neg), ("SIN", torch.sin),
                   ("COS", torch.cos), ("FLOOR", torch.floor), ("CEIL", torch.ceil), ("ROUND", torch.round), ("ELU", F.elu),
                   ("HARD_SWISH", F.hardswish), ("LOGICAL_NOT", torch.logical_not), ("ZEROS_LIKE", torch.zeros_like),
                   ("LOG_SOFTMAX", lambda x: torch.log_softmax(x, -1)), ("DEQUANTIZE", lambda x: x.float()),
                   ("SHAPE", lambda x: torch.tensor(list(x.shape), dtype=torch.int32, device=x.device)),
                   ("RANK", lambda x: torch.tensor(x.dim(), dtype=torch.int32, device=x.device))):
        unary(nm, fn)

    @reg("GELU")
    def gelu(x, approximate=False, **kw):
        return F.gelu(x, approximate="tanh" if approximate else "none")

    @reg("LEAKY_RELU")
    def leaky(x, alpha=0.0, **kw):
        return F.leaky_relu(x, alpha)

    @reg("PRELU")
    def prelu(x, alpha, **kw):
        return torch.where(x >= 0, x, x * alpha.to(x.dtype))

    @reg("L2_NORMALIZATION")
    def l2norm(x, fused_activation_function=0, **kw):
        return _fused(x * torch.rsqrt(torch.clamp((x * x).sum(-1, keepdim=True), min=1e-12)), fused_activation_function)

    @reg("SOFTMAX")
    def softmax(x, beta=1.0, **kw):
        return torch.softmax(x * (beta if beta else 1.0), -1)

    @reg("CONCATENATION")
    def concat(*xs, axis=0, fused_activation_function=0, **kw):
        return _fused(torch.cat(xs, axis), fused_activation_function)

    @reg("RESHAPE")
    def reshape(x, shape=None, new_shape=None, **kw):
        return x.reshape(_ints(shape) if shape is not None else list(new_shape))

    def reducer(name, fn):
        @reg(name)
        def f(x, axes, keep_dims=False, **kw):
            ax = tuple(sorted({a % x.dim() for a in _ints(axes)}))
            return fn(x, ax, bool(keep_dims)) if ax else x
    reducer("MEAN", lambda x, ax, k: x.mean(ax, keepdim=k)); reducer("SUM", lambda x, ax, k: x.sum(ax, keepdim=k))
    reducer("REDUCE_MAX", lambda x, ax, k: x.amax(ax, keepdim=k)); reducer("REDUCE_MIN", lambda x, ax, k: x.amin(ax, keepdim=k))

    @reg("REDUCE_PROD")
    def reduce_prod(x, axes, keep_dims=False, **kw):
        for a in sorted({a % x.dim() for a in _ints(axes)}, reverse=True):
            x = x.prod(a, keepdim=True)
        return x if keep_dims else x.squeeze(tuple(sorted({a % x.dim() for a in _ints(axes)})))

    def _pad(x, paddings, value):
        p = paddings.reshape(-1, 2).tolist()
        flat = []
        for lo, hi in reversed(p):
            flat += [int(lo), int(hi)]
        return F.pad(x, flat, value=value)

    @reg("PAD")
    def pad(x, paddings, **kw): return _pad(x, paddings, 0.0)

    @reg("PADV2")
    def padv2(x, paddings, value, **kw): return _pad(x, paddings, float(value.reshape(-1)[0]))

    @reg("MIRROR_PAD")
    def mirror_pad(x, paddings, mode=0, **kw):
        off = 1 if mode == 0 else 0                    # REFLECT leaves the edge element out, SYMMETRIC repeats it
        for d, (lo, hi) in enumerate(paddings.reshape(-1, 2).tolist()):
            lo, hi, n = int(lo), int(hi), x.shape[d]
            parts = []
            if lo: parts.append(x.narrow(d, off, lo).flip(d))
            parts.append(x)
            if hi: parts.append(x.narrow(d, n - hi - off, hi).flip(d))
            x = torch.cat(parts, d) if len(parts) > 1 else x
        return x

    @reg("TRANSPOSE")
    def transpose(x, perm, **kw): return x.permute(_ints(perm))

    @reg("SQUEEZE")
    def squeeze(x, squeeze_dims=None, **kw):
        dims = [d % x.dim() for d in (squeeze_dims if squeeze_dims is not None else [])]
        return x.squeeze(tuple(dims)) if dims else x.squeeze()

    @reg("EXPAND_DIMS")
    def expand_dims(x, axis, **kw):
        a = _ints(axis)[0]
        return x.unsqueeze(a if a >= 0 else a + x.dim() + 1)

    @reg("STRIDED_SLICE")
    def strided_slice(x, begin, end, strides, begin_mask=0, end_mask=0, ellipsis_mask=0, new_axis_mask=0, shrink_axis_mask=0, **kw):
        b, e, s = _ints(begin), _ints(end), _ints(strides)
        idx, dim = [], 0
        n_real = sum(1 for i in range(len(b)) if not ((new_axis_mask >> i) & 1 or (ellipsis_mask >> i) & 1))
        for i in range(len(b)):
            if (ellipsis_mask >> i) & 1:
                fill = x.dim() - n_real
                idx += [slice(None)] * fill
                dim += fill
            elif (new_axis_mask >> i) & 1:
                idx.append(None)
            elif (shrink_axis_mask >> i) & 1:
                idx.append(b[i])
                dim += 1
            else:
                lo = None if (begin_mask >> i) & 1 else b[i]
                hi = None if (end_mask >> i) & 1 else e[i]
                if s[i] < 0:                           # tensors have no negative-step views: take the range forwards and flip
                    n = x.shape[dim]
                    lo_ = n - 1 if lo is None else (lo + n if lo < 0 else min(lo, n - 1))
                    hi_ = -1 if hi is None else (hi + n if hi < 0 else hi)
                    sel = torch.arange(lo_, hi_, s[i], device=x.device)
                    idx.append(sel)
                else:
                    idx.append(slice(lo, hi, s[i]))
                dim += 1
        return x[tuple(idx)]

    @reg("SLICE")
    def slice_(x, begin, size, **kw):
        idx = tuple(slice(b, None if n < 0 else b + n) for b, n in zip(_ints(begin), _ints(size)))
        return x[idx]

    @reg("GATHER")
    def gather(x, indices, axis=0, batch_dims=0, **kw):
        if batch_dims:
            raise NotImplementedError("GATHER with batch_dims")
        return torch.index_select(x, axis, indices.reshape(-1).long()).reshape(*x.shape[:axis % x.dim()], *indices.shape, *x.shape[axis % x.dim() + 1:])

    @reg("GATHER_ND")
    def gather_nd(x, indices, **kw):
        k = indices.shape[-1]
        return x[tuple(indices[..., j].long() for j in range(k))]

    @reg("EMBEDDING_LOOKUP")
    def embedding_lookup(ids, tbl, **kw): return tbl[ids.long()]

    def _resize(x, size, mode, align_corners, half_pixel_centers):
        oh, ow = _ints(size)
        n, h, w, c = x.shape
        def src(o, i):
            d = torch.arange(o, device=x.device, dtype=torch.float32)
            if align_corners and o > 1:
                return d * ((i - 1) / (o - 1))
            return (d + 0.5) * (i / o) - 0.5 if half_pixel_centers else d * (i / o)
        sy, sx = src(oh, h), src(ow, w)
        if mode == "nearest":
            rnd = (lambda v: torch.floor(v + 0.5)) if (align_corners or half_pixel_centers) else torch.floor
            iy = rnd(sy).clamp(0, h - 1).long()
            ix = rnd(sx).clamp(0, w - 1).long()
            return x[:, iy][:, :, ix]
        sy, sx = sy.clamp(min=0), sx.clamp(min=0)
        y0, x0 = sy.floor().clamp(max=h - 1).long(), sx.floor().clamp(max=w - 1).long()
        y1, x1 = (y0 + 1).clamp(max=h - 1), (x0 + 1).clamp(max=w - 1)
        fy, fx = (sy - y0).reshape(1, -1, 1, 1).to(x.dtype), (sx - x0).reshape(1, 1, -1, 1).to(x.dtype)
        top = x[:, y0][:, :, x0] * (1 - fx) + x[:, y0][:, :, x1] * fx
        bot = x[:, y1][:, :, x0] * (1 - fx) + x[:, y1][:, :, x1] * fx
        return top * (1 - fy) + bot * fy

    @reg("RESIZE_BILINEAR")
    def resize_bilinear(x, size, align_corners=False, half_pixel_centers=False, **kw):
        return _resize(x, size, "bilinear", align_corners, half_pixel_centers)

    @reg("RESIZE_NEAREST_NEIGHBOR")
    def resize_nearest(x, size, align_corners=False, half_pixel_centers=False, **kw):
        return _resize(x, size, "nearest", align_corners, half_pixel_centers)

    @reg("CAST")
    def cast(x, in_data_type=0, out_data_type=0, **kw): return x.to(_TENSOR_TYPES[out_data_type])

    @reg("PACK")
    def pack(*xs, values_count=0, axis=0, **kw): return torch.stack(xs, axis)

    @reg("UNPACK", n_out=-1)
    def unpack(x, num=0, axis=0, **kw): return tuple(x.unbind(axis))

    @reg("SPLIT", n_out=-1)
    def split(axis, x, num_splits=1, **kw):
        a = _ints(axis)[0]
        return tuple(x.chunk(num_splits, a))

    @reg("SPLIT_V", n_out=-1)
    def split_v(x, sizes, axis, num_splits=1, **kw):
        a = _ints(axis)[0] % x.dim()
        sz = _ints(sizes)
        if -1 in sz:
            sz[sz.index(-1)] = x.shape[a] - (sum(sz) + 1)
        return tuple(x.split(sz, a))

    @reg("TILE")
    def tile(x, multiples, **kw): return x.repeat(*_ints(multiples))

    @reg("ARG_MAX")
    def arg_max(x, axis, output_type=4, **kw): return x.argmax(_ints(axis)[0]).to(_TENSOR_TYPES.get(output_type, torch.int64))

    @reg("ARG_MIN")
    def arg_min(x, axis, output_type=4, **kw): return x.argmin(_ints(axis)[0]).to(_TENSOR_TYPES.get(output_type, torch.int64))

    @reg("SELECT")
    def select(c, a, b, **kw):
        if c.dim() == 1 and a.dim() > 1:               # the rank-1 form selects whole rows
            c = c.reshape(-1, *([1] * (a.dim() - 1)))
        return torch.where(c, a, b)

    @reg("SELECT_V2")
    def select_v2(c, a, b, **kw): return torch.where(c, a, b)

    @reg("ONE_HOT")
    def one_hot(indices, depth, on, off, axis=-1, **kw):
        d = _ints(depth)[0]
        oh = F.one_hot(indices.long(), d).bool()
        if axis not in (-1, indices.dim()):
            oh = oh.movedim(-1, axis)
        return torch.where(oh, on.reshape(()), off.reshape(()))

    @reg("FILL")
    def fill(dims, value, **kw): return value.reshape(()).expand(*_ints(dims)).clone()

    @reg("RANGE")
    def range_(start, limit, delta, **kw):
        return torch.arange(start.item(), limit.item(), delta.item(), dtype=start.dtype, device=start.device)

    @reg("SPACE_TO_DEPTH")
    def space_to_depth(x, block_size=1, **kw):
        n, h, w, c = x.shape
        b = block_size
        return x.reshape(n, h // b, b, w // b, b, c).permute(0, 1, 3, 2, 4, 5).reshape(n, h // b, w // b, b * b * c)

    @reg("DEPTH_TO_SPACE")
    def depth_to_space(x, block_size=1, **kw):
        n, h, w, c = x.shape
        b = block_size
        return x.reshape(n, h, w, b, b, c // (b * b)).permute(0, 1, 3, 2, 4, 5).reshape(n, h * b, w * b, c // (b * b))

    @reg("REVERSE_V2")
    def reverse(x, axes, **kw): return x.flip(_ints(axes))

    @reg("CUMSUM")
    def cumsum(x, axis, exclusive=False, reverse=False, **kw):
        a = _ints(axis)[0]
        y = x.flip(a) if reverse else x
        c = y.cumsum(a)
        if exclusive:
            c = c - y
        return c.flip(a) if reverse else c

    @reg("ADD_N")
    def add_n(*xs, **kw):
        out = xs[0]
        for v in xs[1:]:
            out = out + v
        return out

    @reg("L2_POOL_2D")
    def l2_pool(x, padding=0, stride_w=1, stride_h=1, filter_width=1, filter_height=1, fused_activation_function=0, **kw):
        return avg_pool(x * x, padding, stride_w, stride_h, filter_width, filter_height, 0).sqrt() if not fused_activation_function else \
            _fused(avg_pool(x * x, padding, stride_w, stride_h, filter_width, filter_height, 0).sqrt(), fused_activation_function)

    @reg("SPACE_TO_BATCH_ND")
    def space_to_batch(x, block_shape, paddings, **kw):
        bs, pd = _ints(block_shape), paddings.reshape(-1, 2).tolist()
        m = len(bs)
        flat = []
        for d in reversed(range(x.dim())):
            lo, hi = (pd[d - 1] if 1 <= d <= m else (0, 0))
            flat += [int(lo), int(hi)]
        x = F.pad(x, flat)
        n, rest = x.shape[0], list(x.shape[1 + m:])
        shp = [n]
        for i in range(m):
            shp += [x.shape[1 + i] // bs[i], bs[i]]
        x = x.reshape(shp + rest).permute([2 + 2 * i for i in range(m)] + [0] + [1 + 2 * i for i in range(m)] + list(range(1 + 2 * m, 1 + 2 * m + len(rest))))
        prod = 1
        for b in bs:
            prod *= b
        return x.reshape([n * prod] + [shp[1 + 2 * i] for i in range(m)] + rest)

    @reg("BATCH_TO_SPACE_ND")
    def batch_to_space(x, block_shape, crops, **kw):
        bs, cr = _ints(block_shape), crops.reshape(-1, 2).tolist()
        m = len(bs)
        prod = 1
        for b in bs:
            prod *= b
        n, rest = x.shape[0] // prod, list(x.shape[1 + m:])
        x = x.reshape(bs + [n] + list(x.shape[1:1 + m]) + rest)
        perm = [m]
        for i in range(m):
            perm += [m + 1 + i, i]
        x = x.permute(perm + list(range(2 * m + 1, 2 * m + 1 + len(rest))))
        x = x.reshape([n] + [x.shape[1 + 2 * i] * x.shape[2 + 2 * i] for i in range(m)] + rest)
        return x[tuple([slice(None)] + [slice(int(cr[i][0]), x.shape[1 + i] - int(cr[i][1])) for i in range(m)])]

    @reg("TOPK_V2", n_out=2)
    def topk(x, k, **kw):
        v, i = torch.topk(x, _ints(k)[0], dim=-1)
        return v, i.to(torch.int32)

    @reg("SPARSE_TO_DENSE")
    def sparse_to_dense(indices, output_shape, values, default_value, **kw):
        out = torch.full(_ints(output_shape), default_value.item(), dtype=values.dtype)
        idx = indices.long().reshape(-1, 1) if indices.dim() < 2 else indices.long()
        out[tuple(idx[:, j] for j in range(idx.shape[1]))] = values if values.dim() else values.expand(idx.shape[0])
        return out

    reducer("REDUCE_ANY", lambda x, ax, k: x.bool().sum(ax, keepdim=k) > 0)
    reducer("REDUCE_ALL", lambda x, ax, k: (~x.bool()).sum(ax, keepdim=k) == 0)

    @reg("WHERE")
    def where(c, a=None, b=None, **kw): return torch.nonzero(c).to(torch.int64) if a is None else torch.where(c.bool(), a, b)

    @reg("MATRIX_DIAG")
    def matrix_diag(d, **kw): return torch.diag_embed(d)

    @reg("MATRIX_SET_DIAG")
    def matrix_set_diag(x, d, **kw):
        out = x.clone()
        out.diagonal(0, -2, -1).copy_(d)
        return out

    @reg("SCATTER_ND")
    def scatter_nd(indices, updates, shape, **kw):
        out = torch.zeros(_ints(shape), dtype=updates.dtype)
        return out.index_put(tuple(indices[..., j].long() for j in range(indices.shape[-1])), updates, accumulate=True)

    def segment(name, kind, sorted_ids):
        @reg(name)
        def f(data, ids, num=None, **kw):
            ids = ids.long()
            n = _ints(num)[0] if num is not None else int(ids.max()) + 1
            tail = list(data.shape[ids.dim():])
            flat, idx = data.reshape(-1, *tail), ids.reshape(-1)
            keep = idx >= 0
            flat, idx = flat[keep], idx[keep]
            ix = idx.reshape(-1, *([1] * len(tail))).expand_as(flat)
            if kind == "sum":
                return torch.zeros([n] + tail, dtype=data.dtype).scatter_add(0, ix, flat)
            if kind == "prod":
                return torch.ones([n] + tail, dtype=data.dtype).scatter_reduce(0, ix, flat, "prod")
            lim = torch.finfo(data.dtype) if data.dtype.is_floating_point else torch.iinfo(data.dtype)
            return torch.full([n] + tail, lim.min if kind == "max" else lim.max, dtype=data.dtype).scatter_reduce(0, ix, flat, "amax" if kind == "max" else "amin")
    segment("SEGMENT_SUM", "sum", True); segment("UNSORTED_SEGMENT_SUM", "sum", False); segment("UNSORTED_SEGMENT_PROD", "prod", False)
    segment("UNSORTED_SEGMENT_MAX", "max", False); segment("UNSORTED_SEGMENT_MIN", "min", False)

    @reg("BROADCAST_TO")
    def broadcast_to(x, shape, **kw): return x.expand(_ints(shape)).contiguous()

    @reg("BROADCAST_ARGS")
    def broadcast_args(a, b, **kw): return torch.tensor(list(torch.broadcast_shapes(tuple(_ints(a)), tuple(_ints(b)))), dtype=a.dtype)

    @reg("RELU_0_TO_1")
    def relu01(x, **kw): return x.clamp(0, 1)

    @reg("ATAN2")
    def atan2(y, x, **kw): return torch.atan2(y, x)

    @reg("SIGN")
    def sign(x, **kw): return torch.sign(x)

    return ops


_OPS = None


def _register():
    global _OPS
    from ..ops.registry import has, op
    if _OPS is None:
        _OPS = _tflite_ops()
    if has("tflite.ADD"):
        return
    for name, (fn, n_out) in _OPS.items():
        op("tflite." + name, n_out=n_out, group="tflite_import")(fn)


def supportedOps():
    _register()
    return sorted(_OPS)


# ----------------------------------------------------------------------------- model -> SameDiff
def _dequantise(t, q):
    scale = q.get("scale") if q else None
    if scale is None or len(scale) == 0:
        return t
    scale = torch.as_tensor(np.array(scale), dtype=torch.float32)
    zp = q.get("zero_point")
    zp = torch.as_tensor(np.array(zp), dtype=torch.float32) if zp is not None and len(zp) else torch.zeros_like(scale)
    if scale.numel() > 1:
        shp = [1] * t.dim()
        shp[int(q.get("quantized_dimension", 0))] = -1
        scale, zp = scale.reshape(shp), zp.reshape(shp)
    return (t.float() - zp) * scale


class TFLiteImporter:
    def __init__(self, trainable=False):
        self.trainable = trainable

    def runImport(self, path_or_bytes, subgraph=0):
        _register()
        if isinstance(path_or_bytes, (bytes, bytearray, memoryview)):
            data = bytes(path_or_bytes)
        else:
            with open(path_or_bytes, "rb") as f:
                data = f.read()
        if len(data) < 8 or data[4:8] != b"TFL3":
            raise ValueError("not a TensorFlow Lite flatbuffer (file identifier TFL3 missing)")
        model = decode("Model", data, schema=TFL_SCHEMA)
        g = model["subgraphs"][subgraph]
        codes = []
        for oc in model["operator_codes"]:
            code = max(int(oc["builtin_code"]), int(oc["deprecated_builtin_code"]))   # codes < 127 live in the old byte field
            codes.append(oc["custom_code"] if code == 32 else BUILTIN.get(code, f"builtin#{code}"))
        used = [codes[o["opcode_index"]] for o in g["operators"]]
        missing = sorted({c for c in used if c not in _OPS})
        if missing:
            raise NotImplementedError(f"TFLite import: no rule for operators {missing}")
        tensors = g["tensors"]
        produced = {o for op_ in g["operators"] for o in op_["outputs"]}
        sd = SameDiff.create()
        vars_ = {}
        names = {}

        def name_of(i):
            if i not in names:
                n = tensors[i]["name"] or f"tensor_{i}"
                names[i] = n if n not in names.values() else f"{n}_{i}"
            return names[i]

        for i in list(g["inputs"]):
            t = tensors[i]
            q = t.get("quantization")
            if t["type"] not in (0, 1, 10, 2, 4, 6) and q and q.get("scale") is not None and len(q["scale"]):
                raise NotImplementedError("TFLite import: quantised activations (a fully quantised graph) are not supported")
            shape = list(t["shape_signature"]) if t.get("shape_signature") is not None and len(t["shape_signature"]) else list(t["shape"] if t["shape"] is not None else [])
            vars_[i] = sd.placeHolder(name_of(i), _DL4J_TYPES.get(t["type"], DataType.FLOAT), *[int(s) for s in shape])
        for i, t in enumerate(tensors):
            if i in vars_ or i in produced:
                continue
            buf = model["buffers"][t["buffer"]]["data"] if t["buffer"] < len(model["buffers"]) else None
            if buf is None or len(buf) == 0:
                continue
            dt = _TENSOR_TYPES[t["type"]]
            shape = [int(s) for s in (t["shape"] if t["shape"] is not None else [])]
            arr = torch.frombuffer(bytearray(buf), dtype=dt).reshape(shape).clone()
            if dt in (torch.int8, torch.uint8, torch.int16):
                arr = _dequantise(arr, t.get("quantization"))
            elif dt == torch.float16:
                arr = arr.float()
            if self.trainable and arr.is_floating_point() and arr.dim() >= 1:
                vars_[i] = sd.var(name_of(i), arr)
            else:
                vars_[i] = sd.constant(name_of(i), arr)
        for op_ in g["operators"]:
            kind = codes[op_["opcode_index"]]
            ins = [vars_.get(i) if i >= 0 else None for i in op_["inputs"]]
            while ins and ins[-1] is None:
                ins.pop()
            opts = op_.get("builtin_options") or {}
            attrs = {k: (v.tolist() if isinstance(v, np.ndarray) else v) for k, v in opts.items() if v is not None}
            n_out = _OPS[kind][1]
            kw = dict(n_out=len(op_["outputs"])) if n_out == -1 else {}
            out = sd._op("tflite." + kind, ins, **kw, **attrs)
            outs = out if isinstance(out, (list, tuple)) else [out]
            for i, v in zip(op_["outputs"], outs):
                nm = name_of(i)
                if v.name != nm:
                    v = sd.renameVariable(v.name, nm) or sd.getVariable(nm)
                vars_[i] = sd.getVariable(nm) if sd.hasVariable(nm) else v
        self.inputs = [name_of(i) for i in g["inputs"]]
        self.outputs = [name_of(i) for i in g["outputs"]]
        sd.metadata["tflite.inputs"] = ",".join(self.inputs)
        sd.metadata["tflite.outputs"] = ",".join(self.outputs)
        sd.metadata["tflite.description"] = model.get("description") or ""
        return sd


def importTFLite(path_or_bytes, trainable=False, subgraph=0):
    return TFLiteImporter(trainable).runImport(path_or_bytes, subgraph)
