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


def _ints(t):
    return [int(v) for v in (t.reshape(-1).tolist() if isinstance(t, torch.Tensor) else t)]


def _tf_ops():
    """TensorFlow op type -> (function(inputs..., **attrs), number of outputs; -1 = variable).  Arguments that TensorFlow passes as
    tensors (shapes, axes, paddings, ...) stay tensor inputs, so they may be computed inside the graph."""
    import torch.nn.functional as F

    def strided(x, begin, end, strides, begin_mask=0, end_mask=0, ellipsis_mask=0, new_axis_mask=0, shrink_axis_mask=0, **kw):
        b, e, st = _ints(begin), _ints(end), _ints(strides)
        idx, dim = [], 0
        for i in range(len(b)):
            if ellipsis_mask >> i & 1:
                idx.append(Ellipsis)
                dim = x.dim() - (len(b) - i - 1 - sum((new_axis_mask >> j) & 1 for j in range(i + 1, len(b))))
                continue
            if new_axis_mask >> i & 1:
                idx.append(None)
                continue
            if shrink_axis_mask >> i & 1:
                idx.append(b[i])
                dim += 1
                continue
            lo = None if begin_mask >> i & 1 else b[i]
            hi = None if end_mask >> i & 1 else e[i]
            if st[i] < 0:                      # torch has no negative steps: flip the axis and mirror the bounds
                n = x.shape[dim]
                lo2 = 0 if lo is None else n - 1 - (lo if lo >= 0 else n + lo)
                hi2 = n if hi is None else n - 1 - (hi if hi >= 0 else n + hi)
                x = x.flip(dim)
                idx.append(slice(lo2, hi2, -st[i]))
            else:
                idx.append(slice(lo, hi, st[i]))
            dim += 1
        return x[tuple(idx)]

    def resize(x, size, mode, align_corners=False, half_pixel_centers=False, **kw):
        h, w = _ints(size)
        y = x.permute(0, 3, 1, 2).float()
        if mode == "nearest":
            if half_pixel_centers or align_corners:
                y = F.interpolate(y, size=(h, w), mode="nearest-exact" if half_pixel_centers else "nearest")
            else:
                ih = (torch.arange(h, device=x.device) * (x.shape[1] / h)).floor().long().clamp(max=x.shape[1] - 1)
                iw = (torch.arange(w, device=x.device) * (x.shape[2] / w)).floor().long().clamp(max=x.shape[2] - 1)
                y = y[:, :, ih][:, :, :, iw]
        elif align_corners:
            y = F.interpolate(y, size=(h, w), mode="bilinear", align_corners=True)
        elif half_pixel_centers:
            y = F.interpolate(y, size=(h, w), mode="bilinear", align_corners=False)
        else:                                  # TensorFlow 1.x default: source = destination * scale, no half-pixel offset
            sy, sx = x.shape[1] / h, x.shape[2] / w
            fy, fx = torch.arange(h, device=x.device) * sy, torch.arange(w, device=x.device) * sx
            y0, x0 = fy.floor().long().clamp(max=x.shape[1] - 1), fx.floor().long().clamp(max=x.shape[2] - 1)
            y1, x1 = (y0 + 1).clamp(max=x.shape[1] - 1), (x0 + 1).clamp(max=x.shape[2] - 1)
            wy, wx = (fy - y0).reshape(1, 1, -1, 1), (fx - x0).reshape(1, 1, 1, -1)
            top = y[:, :, y0][:, :, :, x0] * (1 - wx) + y[:, :, y0][:, :, :, x1] * wx
            bot = y[:, :, y1][:, :, :, x0] * (1 - wx) + y[:, :, y1][:, :, :, x1] * wx
            y = top * (1 - wy) + bot * wy
        return y.permute(0, 2, 3, 1).to(x.dtype if mode == "nearest" else torch.float32)

    def conv_t(out_shape, w, dy, strides=(1, 1, 1, 1), padding="SAME", data_format="NHWC", **kw):
        nhwc = data_format == "NHWC"
        g = dy.permute(0, 3, 1, 2) if nhwc else dy
        s = (strides[1], strides[2]) if nhwc else (strides[2], strides[3])
        osz = _ints(out_shape)
        oh, ow = (osz[1], osz[2]) if nhwc else (osz[2], osz[3])
        wt = w.permute(3, 2, 0, 1)                   # HWIO (I = output channels of the transpose) -> [in=O, out=I, kh, kw]
        kh, kw_ = wt.shape[2:]
        if padding == "SAME":
            ph = max((g.shape[2] - 1) * s[0] + kh - oh, 0)
            pw_ = max((g.shape[3] - 1) * s[1] + kw_ - ow, 0)
            y = F.conv_transpose2d(g, wt.to(g.dtype), None, s, 0)
            y = y[:, :, ph // 2:ph // 2 + oh, pw_ // 2:pw_ // 2 + ow]
        else:
            y = F.conv_transpose2d(g, wt.to(g.dtype), None, s, 0)
            y = F.pad(y, (0, ow - y.shape[3], 0, oh - y.shape[2]))
        return y.permute(0, 2, 3, 1) if nhwc else y

    def sd_(x, bs, to_depth, data_format="NHWC", **kw):
        y = x.permute(0, 3, 1, 2) if data_format == "NHWC" else x
        if to_depth:                                 # TensorFlow's channel order: (block row, block column, channel)
            n, c, h, w = y.shape
            y = y.reshape(n, c, h // bs, bs, w // bs, bs).permute(0, 3, 5, 1, 2, 4).reshape(n, c * bs * bs, h // bs, w // bs)
        else:
            n, c, h, w = y.shape
            y = y.reshape(n, bs, bs, c // (bs * bs), h, w).permute(0, 3, 4, 1, 5, 2).reshape(n, c // (bs * bs), h * bs, w * bs)
        return y.permute(0, 2, 3, 1) if data_format == "NHWC" else y

    def xent_sparse(logits, labels, **kw):
        ls = torch.log_softmax(logits.float(), -1)
        loss = -ls.gather(-1, labels.long().unsqueeze(-1)).squeeze(-1)
        return loss, torch.softmax(logits.float(), -1) - F.one_hot(labels.long(), logits.shape[-1]).float()

    def xent(logits, labels, **kw):
        ls = torch.log_softmax(logits.float(), -1)
        return -(labels * ls).sum(-1), torch.softmax(logits.float(), -1) - labels

    def lrn(x, depth_radius=5, bias=1.0, alpha=1.0, beta=0.5, **kw):
        sq = (x * x).permute(0, 3, 1, 2)
        pad = F.pad(sq, (0, 0, 0, 0, depth_radius, depth_radius))
        win = sum(pad[:, i:i + sq.shape[1]] for i in range(2 * depth_radius + 1))
        return x / (bias + alpha * win.permute(0, 2, 3, 1)) ** beta

    def gather(x, idx, axis=0, batch_dims=0, **kw):
        axis = int(axis) % x.dim()
        if batch_dims:
            return torch.stack([gather(xb, ib, axis - 1, batch_dims - 1) for xb, ib in zip(x, idx)])
        return x.index_select(axis, idx.reshape(-1).long()).reshape(*x.shape[:axis], *idx.shape, *x.shape[axis + 1:])

    def gather_nd(x, idx, **kw):
        idx = idx.long()
        return x[tuple(idx[..., i] for i in range(idx.shape[-1]))]

    def one_hot(idx, depth, on, off, axis=-1, **kw):
        d = int(depth)
        oh = F.one_hot(idx.long().clamp(0, max(d - 1, 0)), d).bool() & ((idx >= 0) & (idx < d)).unsqueeze(-1)
        y = torch.where(oh, on, off)
        return y if axis in (-1, idx.dim()) else y.movedim(-1, int(axis))

    def cumsum(x, axis, exclusive=False, reverse=False, **kw):
        a = int(axis)
        if reverse:
            x = x.flip(a)
        y = x.cumsum(a)
        if exclusive:
            y = y - x
        return y.flip(a) if reverse else y

    def red(fn):
        def f(x, axis, keep_dims=False, **kw):
            ax = tuple(_ints(axis))
            if not ax and isinstance(axis, torch.Tensor) and axis.numel() == 0:
                return x
            return fn(x, ax, bool(keep_dims))
        return f

    def unpack(x, axis=0, num=None, **kw): return tuple(x.unbind(int(axis)))
    def split(axis, x, num_split=1, **kw): return tuple(x.chunk(int(num_split), int(axis)))
    def split_v(x, sizes, axis, num_split=None, **kw):
        sz = _ints(sizes)
        if -1 in sz:
            sz[sz.index(-1)] = x.shape[int(axis)] - sum(v for v in sz if v >= 0)
        return tuple(x.split(sz, int(axis)))

    def pad(x, paddings, value=0.0, mode="constant"):
        p = paddings.reshape(-1, 2).tolist()
        if mode == "constant":
            flat = []
            for lo, hi in reversed(p):
                flat += [int(lo), int(hi)]
            return F.pad(x, flat, value=float(value))
        y = x
        for d, (lo, hi) in enumerate(p):           # REFLECT excludes the border element, SYMMETRIC repeats it
            lo, hi, n = int(lo), int(hi), y.shape[d]
            off = 1 if mode == "reflect" else 0
            front = y.narrow(d, off, lo).flip(d) if lo else None
            back = y.narrow(d, n - hi - off, hi).flip(d) if hi else None
            y = torch.cat([t for t in (front, y, back) if t is not None], d)
        return y

    def bmm(x, y, adj_x=False, adj_y=False, **kw):
        return torch.matmul(x.transpose(-1, -2) if adj_x else x, y.transpose(-1, -2) if adj_y else y)

    def band_part(x, lower, upper, **kw):
        lo, up = int(lower), int(upper)
        r = torch.arange(x.shape[-2], device=x.device)[:, None]
        c = torch.arange(x.shape[-1], device=x.device)[None, :]
        keep = ((lo < 0) | (r - c <= lo)) & ((up < 0) | (c - r <= up))
        return x * keep.to(x.dtype)

    def scatter_nd(indices, updates, shape, **kw):
        out = torch.zeros(_ints(shape), dtype=updates.dtype, device=updates.device)
        k = indices.shape[-1]
        idx = tuple(indices[..., j].long() for j in range(k))
        return out.index_put(idx, updates, accumulate=True)               # duplicate indices add up, as in TensorFlow

    def space_to_batch_nd(x, block_shape, paddings, **kw):
        bs, pd = _ints(block_shape), paddings.reshape(-1, 2).tolist()
        m = len(bs)
        flat = []
        for d in reversed(range(x.dim())):
            lo, hi = (pd[d - 1] if 1 <= d <= m else (0, 0))
            flat += [int(lo), int(hi)]
        x = F.pad(x, flat)
        n = x.shape[0]
        shp = [n]
        for i in range(m):
            shp += [x.shape[1 + i] // bs[i], bs[i]]
        rest = list(x.shape[1 + m:])
        x = x.reshape(shp + rest)
        perm = [2 + 2 * i for i in range(m)] + [0] + [1 + 2 * i for i in range(m)] + list(range(1 + 2 * m, 1 + 2 * m + len(rest)))
        x = x.permute(perm)
        return x.reshape([n * int(np.prod(bs))] + [shp[1 + 2 * i] for i in range(m)] + rest)

    def batch_to_space_nd(x, block_shape, crops, **kw):
        bs, cr = _ints(block_shape), crops.reshape(-1, 2).tolist()
        m = len(bs)
        n = x.shape[0] // int(np.prod(bs))
        rest = list(x.shape[1 + m:])
        x = x.reshape(bs + [n] + list(x.shape[1:1 + m]) + rest)
        perm = [m]
        for i in range(m):
            perm += [m + 1 + i, i]
        perm += list(range(2 * m + 1, 2 * m + 1 + len(rest)))
        x = x.permute(perm)
        x = x.reshape([n] + [x.shape[1 + 2 * i] * x.shape[2 + 2 * i] for i in range(m)] + rest)
        idx = [slice(None)] + [slice(int(cr[i][0]), x.shape[1 + i] - int(cr[i][1])) for i in range(m)]
        return x[tuple(idx)]

    def _same3(size, k, st, dl):
        eff = (k - 1) * dl + 1
        total = max((-(-size // st) - 1) * st + eff - size, 0)
        return total // 2, total - total // 2

    def conv3d(x, w, strides=(1, 1, 1, 1, 1), padding="VALID", dilations=(1, 1, 1, 1, 1), data_format="NDHWC", **kw):
        padding = padding.decode() if isinstance(padding, bytes) else padding
        cl = (data_format.decode() if isinstance(data_format, bytes) else data_format) == "NDHWC"
        xn = x.permute(0, 4, 1, 2, 3) if cl else x
        st = list(strides[1:4]) if cl else list(strides[2:5])
        dl = list(dilations[1:4]) if cl else list(dilations[2:5])
        wk = w.permute(4, 3, 0, 1, 2)                                        # DHWIO -> OIDHW
        if padding == "SAME":
            flat = []
            for d in (2, 1, 0):
                lo, hi = _same3(xn.shape[2 + d], wk.shape[2 + d], st[d], dl[d])
                flat += [lo, hi]
            xn = F.pad(xn, flat)
        y = F.conv3d(xn, wk, None, st, 0, dl)
        return y.permute(0, 2, 3, 4, 1) if cl else y

    def pool3d(x, kind, ksize=(1, 1, 1, 1, 1), strides=(1, 1, 1, 1, 1), padding="VALID", data_format="NDHWC", **kw):
        padding = padding.decode() if isinstance(padding, bytes) else padding
        cl = (data_format.decode() if isinstance(data_format, bytes) else data_format) == "NDHWC"
        xn = x.permute(0, 4, 1, 2, 3) if cl else x
        k = list(ksize[1:4]) if cl else list(ksize[2:5])
        st = list(strides[1:4]) if cl else list(strides[2:5])
        if padding == "SAME":
            flat = []
            for d in (2, 1, 0):
                lo, hi = _same3(xn.shape[2 + d], k[d], st[d], 1)
                flat += [lo, hi]
            if kind == "max":
                xn = F.pad(xn, flat, value=float("-inf"))
                y = F.max_pool3d(xn, k, st)
            else:
                ones = F.avg_pool3d(F.pad(torch.ones_like(xn[:1, :1]), flat), k, st)
                y = F.avg_pool3d(F.pad(xn, flat), k, st) / ones
        else:
            y = F.max_pool3d(xn, k, st) if kind == "max" else F.avg_pool3d(xn, k, st)
        return y.permute(0, 2, 3, 4, 1) if cl else y

    def nms_v3(boxes, scores, max_output_size, iou_threshold, score_threshold, **kw):
        m, it, stt = int(max_output_size), float(iou_threshold), float(score_threshold)
        y1, x1, y2, x2 = boxes.unbind(1)
        x1, x2 = torch.minimum(x1, x2), torch.maximum(x1, x2)
        y1, y2 = torch.minimum(y1, y2), torch.maximum(y1, y2)
        area = (x2 - x1) * (y2 - y1)
        keep = []
        for i in scores.argsort(descending=True).tolist():
            if float(scores[i]) <= stt or len(keep) >= m:
                break
            ok = True
            for j in keep:
                inter = (torch.minimum(x2[i], x2[j]) - torch.maximum(x1[i], x1[j])).clamp(min=0) * \
                        (torch.minimum(y2[i], y2[j]) - torch.maximum(y1[i], y1[j])).clamp(min=0)
                union = area[i] + area[j] - inter
                if float(union) > 0 and float(inter / union) > it:
                    ok = False
                    break
            if ok:
                keep.append(i)
        return torch.tensor(keep, dtype=torch.int32)

    T = {
        "Less": (lambda a, b, **k: a < b, 1), "LessEqual": (lambda a, b, **k: a <= b, 1), "Greater": (lambda a, b, **k: a > b, 1),
        "GreaterEqual": (lambda a, b, **k: a >= b, 1), "Equal": (lambda a, b, **k: a == b, 1), "NotEqual": (lambda a, b, **k: a != b, 1),
        "LogicalAnd": (lambda a, b, **k: a & b, 1), "LogicalOr": (lambda a, b, **k: a | b, 1), "LogicalNot": (lambda a, **k: ~a, 1),
        "Select": (lambda c, a, b, **k: torch.where(c.reshape(list(c.shape) + [1] * (a.dim() - c.dim())) if c.dim() < a.dim() else c, a, b), 1),
        "SelectV2": (lambda c, a, b, **k: torch.where(c, a, b), 1),
        "FloorDiv": (lambda a, b, **k: torch.div(a, b, rounding_mode="floor"), 1), "FloorMod": (lambda a, b, **k: torch.remainder(a, b), 1),
        "Mod": (lambda a, b, **k: torch.fmod(a, b), 1), "TruncateDiv": (lambda a, b, **k: torch.div(a, b, rounding_mode="trunc"), 1),
        "Range": (lambda a, b, c, **k: torch.arange(a.item(), b.item(), c.item(), dtype=a.dtype, device=a.device), 1),
        "Fill": (lambda sh, v, **k: torch.full(_ints(sh), v.item(), dtype=v.dtype, device=v.device), 1),
        "ZerosLike": (lambda x, **k: torch.zeros_like(x), 1), "OnesLike": (lambda x, **k: torch.ones_like(x), 1),
        "Tile": (lambda x, m, **k: x.repeat(*_ints(m)), 1),
        "Slice": (lambda x, b, sz, **k: x[tuple(slice(bi, None if si < 0 else bi + si) for bi, si in zip(_ints(b), _ints(sz)))], 1),
        "StridedSlice": (strided, 1), "Split": (split, -1), "SplitV": (split_v, -1), "Unpack": (unpack, -1),
        "Gather": (lambda x, i, **k: gather(x, i, 0), 1), "GatherV2": (lambda x, i, ax, batch_dims=0, **k: gather(x, i, int(ax), batch_dims), 1),
        "GatherNd": (gather_nd, 1), "OneHot": (one_hot, 1),
        "TopKV2": (lambda x, kk, sorted=True, **k: tuple(t if j == 0 else t.to(torch.int32) for j, t in enumerate(torch.topk(x, int(kk), sorted=True))), 2),
        "Cumsum": (cumsum, 1), "Cumprod": (lambda x, ax, **k: x.cumprod(int(ax)), 1),
        "Sin": (lambda x, **k: x.sin(), 1), "Cos": (lambda x, **k: x.cos(), 1), "Tan": (lambda x, **k: x.tan(), 1),
        "Asin": (lambda x, **k: x.asin(), 1), "Acos": (lambda x, **k: x.acos(), 1), "Atan": (lambda x, **k: x.atan(), 1),
        "Sinh": (lambda x, **k: x.sinh(), 1), "Cosh": (lambda x, **k: x.cosh(), 1), "Atan2": (lambda a, b, **k: torch.atan2(a, b), 1),
        "Ceil": (lambda x, **k: x.ceil(), 1), "Round": (lambda x, **k: x.round(), 1), "Rint": (lambda x, **k: x.round(), 1),
        "Sign": (lambda x, **k: x.sign(), 1), "Reciprocal": (lambda x, **k: 1.0 / x, 1), "Inv": (lambda x, **k: 1.0 / x, 1),
        "Log1p": (lambda x, **k: x.log1p(), 1), "Expm1": (lambda x, **k: x.expm1(), 1), "Softsign": (lambda x, **k: x / (1 + x.abs()), 1),
        "IsNan": (lambda x, **k: x.isnan(), 1), "IsInf": (lambda x, **k: x.isinf(), 1), "IsFinite": (lambda x, **k: x.isfinite(), 1),
        "Size": (lambda x, **k: torch.tensor(x.numel(), dtype=torch.int32), 1), "Rank": (lambda x, **k: torch.tensor(x.dim(), dtype=torch.int32), 1),
        "ArgMin": (lambda x, ax, **k: x.argmin(int(ax)), 1),
        "All": (red(lambda x, ax, kd: x.all(ax[0], kd) if len(ax) == 1 else x.float().amin(ax, kd).bool()), 1),
        "Any": (red(lambda x, ax, kd: x.any(ax[0], kd) if len(ax) == 1 else x.float().amax(ax, kd).bool()), 1),
        "BatchMatMul": (bmm, 1), "BatchMatMulV2": (bmm, 1), "AddN": (lambda *xs, **k: torch.stack(xs).sum(0), 1),
        "Conv2DBackpropInput": (conv_t, 1),
        "ResizeBilinear": (lambda x, sz, **k: resize(x, sz, "bilinear", **k), 1),
        "ResizeNearestNeighbor": (lambda x, sz, **k: resize(x, sz, "nearest", **k), 1),
        "SpaceToDepth": (lambda x, block_size=2, data_format="NHWC", **k: sd_(x, int(block_size), True, data_format), 1),
        "DepthToSpace": (lambda x, block_size=2, data_format="NHWC", **k: sd_(x, int(block_size), False, data_format), 1),
        "PadV2": (lambda x, p, v, **k: pad(x, p, v.item()), 1),
        "MirrorPad": (lambda x, p, mode="REFLECT", **k: pad(x, p, mode=mode.lower()), 1),
        "ReverseV2": (lambda x, ax, **k: x.flip(_ints(ax)), 1),
        "ClipByValue": (lambda x, lo, hi, **k: torch.minimum(torch.maximum(x, lo), hi), 1),
        "L2Loss": (lambda x, **k: (x * x).sum() / 2, 1), "LRN": (lrn, 1),
        "IdentityN": (lambda *xs, **k: tuple(xs), -1), "Snapshot": (lambda x, **k: x, 1), "PreventGradient": (lambda x, **k: x.detach(), 1),
        "SparseSoftmaxCrossEntropyWithLogits": (xent_sparse, 2), "SoftmaxCrossEntropyWithLogits": (xent, 2),
        "Where": (lambda c, **k: c.nonzero(), 1), "Swish": (lambda x, **k: x * torch.sigmoid(x), 1),
        "BroadcastTo": (lambda x, sh, **k: x.broadcast_to(_ints(sh)), 1), "Einsum": (lambda *xs, equation="", **k: torch.einsum(equation, *xs), 1),
        "MatrixDiag": (lambda x, **k: torch.diag_embed(x), 1), "MatrixDiagPart": (lambda x, **k: torch.diagonal(x, dim1=-2, dim2=-1), 1),
        "Tanh": (lambda x, **k: x.tanh(), 1),
        "Assert": (lambda cond, *data, **k: cond, 1),                       # checked at import time only when constant; a no-op at run time
        "ShapeN": (lambda *xs, out_type=None, **k: tuple(torch.tensor(list(x.shape), dtype=torch.int32) for x in xs), -1),
        "MatrixBandPart": (band_part, 1), "ScatterNd": (scatter_nd, 1),
        "SpaceToBatchND": (space_to_batch_nd, 1), "BatchToSpaceND": (batch_to_space_nd, 1),
        "Conv3D": (conv3d, 1), "MaxPool3D": (lambda x, **k: pool3d(x, "max", **k), 1), "AvgPool3D": (lambda x, **k: pool3d(x, "avg", **k), 1),
        "RandomUniform": (lambda shape, dtype=None, seed=0, seed2=0, **k: torch.rand(_ints(shape)), 1),
        "NonMaxSuppressionV3": (nms_v3, 1),
    }
    T.update(_tf_ops_more(T, nms_v3))
    return T


def _tf_ops_more(T, nms_v3):
    """Second table of GraphDef operators: special functions, bitwise, segment / scatter / partition ops, linear algebra,
    random ops, image ops and the older spellings of ops the first table already has."""
    import torch.nn.functional as F

    def s_(v):
        return v.decode() if isinstance(v, bytes) else v

    def segment(kind):
        def f(data, ids, num=None, **kw):
            ids = ids.long()
            n = int(num) if num is not None else (int(ids.max()) + 1 if ids.numel() else 0)
            shape = [n] + list(data.shape[ids.dim():])
            flat = data.reshape(-1, *data.shape[ids.dim():])
            idx = ids.reshape(-1)
            keep = idx >= 0                                                             # negative ids are dropped (unsorted variants)
            flat, idx = flat[keep], idx[keep]
            ix = idx.reshape(-1, *([1] * (flat.dim() - 1))).expand_as(flat)
            if kind in ("sum", "mean"):
                out = torch.zeros(shape, dtype=data.dtype).scatter_add(0, ix, flat)
                if kind == "mean":
                    cnt = torch.zeros(n, dtype=data.dtype).scatter_add(0, idx, torch.ones_like(idx, dtype=data.dtype)).clamp(min=1)
                    out = out / cnt.reshape(-1, *([1] * (flat.dim() - 1)))
                return out
            if kind == "prod":
                return torch.ones(shape, dtype=data.dtype).scatter_reduce(0, ix, flat, "prod")
            fill = torch.finfo(data.dtype).min if data.dtype.is_floating_point else torch.iinfo(data.dtype).min
            if kind == "min":
                fill = torch.finfo(data.dtype).max if data.dtype.is_floating_point else torch.iinfo(data.dtype).max
            empty = 0 if num is None else fill                                          # sorted variants give 0 for an empty segment
            out = torch.full(shape, fill, dtype=data.dtype).scatter_reduce(0, ix, flat, "amax" if kind == "max" else "amin")
            hit = torch.zeros(n, dtype=torch.bool).index_fill(0, idx, True).reshape(-1, *([1] * (flat.dim() - 1)))
            return torch.where(hit, out, torch.full_like(out, empty))
        return f

    def tensor_scatter(kind):
        def f(x, indices, updates, **kw):
            idx = tuple(indices[..., j].long() for j in range(indices.shape[-1]))
            if kind == "update":
                return x.index_put(idx, updates)
            return x.index_put(idx, updates if kind == "add" else -updates, accumulate=True)
        return f

    def dynamic_partition(data, partitions, num_partitions=2, **kw):
        return tuple(data[partitions == i] for i in range(int(num_partitions)))

    def dynamic_stitch(*args, N=None, **kw):
        n = len(args) // 2
        idx, data = args[:n], args[n:]
        size = max(int(i.max()) + 1 for i in idx if i.numel())
        tail = data[0].shape[idx[0].dim():]
        out = torch.zeros([size] + list(tail), dtype=data[0].dtype)
        for i, d in zip(idx, data):                                                     # later inputs win, as in TensorFlow
            out[i.reshape(-1).long()] = d.reshape(-1, *tail)
        return out

    def fake_quant(x, lo, hi, num_bits=8, narrow_range=False, **kw):
        qmin, qmax = (1 if narrow_range else 0), 2 ** int(num_bits) - 1
        lo, hi = torch.as_tensor(lo, dtype=x.dtype), torch.as_tensor(hi, dtype=x.dtype)
        scale = (hi - lo) / (qmax - qmin)
        zp = qmin - lo / scale                                                          # nudged so that zero is exactly representable
        nz = torch.where(zp < qmin, torch.full_like(zp, qmin), torch.where(zp > qmax, torch.full_like(zp, qmax), torch.round(zp)))
        nlo, nhi = (qmin - nz) * scale, (qmax - nz) * scale
        c = torch.minimum(torch.maximum(x, nlo), nhi)
        return torch.floor((c - nlo) / scale + 0.5) * scale + nlo

    def in_top_k(pred, targets, k, **kw):
        k = int(k)
        t = pred.gather(1, targets.long().reshape(-1, 1))
        return (pred > t).sum(1) < k

    def matrix_set_diag(x, d, k=0, **kw):
        out = x.clone()
        out.diagonal(int(k) if not torch.is_tensor(k) else int(k), -2, -1).copy_(d)
        return out

    def max_pool_argmax(x, ksize=(1, 1, 1, 1), strides=(1, 1, 1, 1), padding="VALID", include_batch_in_index=False, **kw):
        xn = x.permute(0, 3, 1, 2)
        k, st = list(ksize[1:3]), list(strides[1:3])
        if s_(padding) == "SAME":
            ph = max((-(-xn.shape[2] // st[0]) - 1) * st[0] + k[0] - xn.shape[2], 0)
            pw = max((-(-xn.shape[3] // st[1]) - 1) * st[1] + k[1] - xn.shape[3], 0)
            if ph or pw:
                raise NotImplementedError("MaxPoolWithArgmax with SAME padding that pads")
        y, ix = F.max_pool2d(xn, k, st, return_indices=True)                           # ix = h * W + w within a channel plane
        H, W, C = x.shape[1], x.shape[2], x.shape[3]
        c = torch.arange(C).reshape(1, C, 1, 1)
        flat = ix * C + c                                                               # ((h * W) + w) * C + c, the NHWC flat index
        if include_batch_in_index:
            flat = flat + torch.arange(x.shape[0]).reshape(-1, 1, 1, 1) * (H * W * C)
        return y.permute(0, 2, 3, 1), flat.permute(0, 2, 3, 1)

    def resize(mode):
        def f(x, size, align_corners=False, half_pixel_centers=False, **kw):
            h, w = _ints(size)
            xn = x.permute(0, 3, 1, 2).float()
            if mode == "area":
                y = F.adaptive_avg_pool2d(xn, (h, w))
            else:
                y = F.interpolate(xn, size=(h, w), mode="bicubic", align_corners=bool(align_corners))
            return y.permute(0, 2, 3, 1)
        return f

    def crop_and_resize(image, boxes, box_ind, crop_size, method="bilinear", extrapolation_value=0.0, **kw):
        ch, cw = _ints(crop_size)
        N, H, W, C = image.shape
        out = []
        for b, bi in zip(boxes, box_ind.long()):
            y1, x1, y2, x2 = [float(v) for v in b]
            ys = torch.linspace(y1 * (H - 1), y2 * (H - 1), ch) if ch > 1 else torch.tensor([0.5 * (y1 + y2) * (H - 1)])
            xs = torch.linspace(x1 * (W - 1), x2 * (W - 1), cw) if cw > 1 else torch.tensor([0.5 * (x1 + x2) * (W - 1)])
            img = image[bi].float()
            if s_(method) == "nearest":
                yi, xi = ys.round().long().clamp(0, H - 1), xs.round().long().clamp(0, W - 1)
                crop = img[yi][:, xi]
            else:
                y0, x0 = ys.floor().long().clamp(0, H - 1), xs.floor().long().clamp(0, W - 1)
                y1i, x1i = (y0 + 1).clamp(max=H - 1), (x0 + 1).clamp(max=W - 1)
                fy, fx = (ys - y0).reshape(-1, 1, 1), (xs - x0).reshape(1, -1, 1)
                top = img[y0][:, x0] * (1 - fx) + img[y0][:, x1i] * fx
                bot = img[y1i][:, x0] * (1 - fx) + img[y1i][:, x1i] * fx
                crop = top * (1 - fy) + bot * fy
            inside = ((ys >= 0) & (ys <= H - 1)).reshape(-1, 1, 1) & ((xs >= 0) & (xs <= W - 1)).reshape(1, -1, 1)
            out.append(torch.where(inside, crop, torch.full_like(crop, float(extrapolation_value))))
        return torch.stack(out)

    def extract_patches(x, ksizes=(1, 1, 1, 1), strides=(1, 1, 1, 1), rates=(1, 1, 1, 1), padding="VALID", **kw):
        if s_(padding) != "VALID":
            raise NotImplementedError("ExtractImagePatches with SAME padding")
        xn = x.permute(0, 3, 1, 2)
        n, c = xn.shape[:2]
        cols = F.unfold(xn, list(ksizes[1:3]), dilation=list(rates[1:3]), stride=list(strides[1:3]))   # [n, c*kh*kw, L]
        kh, kw_ = ksizes[1], ksizes[2]
        oh = (xn.shape[2] - (kh - 1) * rates[1] - 1) // strides[1] + 1
        cols = cols.reshape(n, c, kh, kw_, oh, -1).permute(0, 4, 5, 2, 3, 1)             # patch depth in (row, col, channel) order
        return cols.reshape(n, oh, cols.shape[2], kh * kw_ * c)

    def rgb_to_hsv(x, **kw):
        r, g, b = x.unbind(-1)
        mx, mn = x.max(-1).values, x.min(-1).values
        d = mx - mn
        s = torch.where(mx > 0, d / mx.clamp(min=1e-30), torch.zeros_like(mx))
        dd = d.clamp(min=1e-30)
        h = torch.where(mx == r, ((g - b) / dd) % 6, torch.where(mx == g, (b - r) / dd + 2, (r - g) / dd + 4)) / 6
        h = torch.where(d == 0, torch.zeros_like(h), h)
        return torch.stack([h, s, mx], -1)

    def hsv_to_rgb(x, **kw):
        h, s, v = x.unbind(-1)
        k = lambda n: (n + h * 6) % 6
        f = lambda n: v - v * s * torch.clamp(torch.minimum(k(n), 4 - k(n)), 0, 1)
        return torch.stack([f(5), f(3), f(1)], -1)

    def adjust_hue(x, delta, **kw):
        hsv = rgb_to_hsv(x)
        return hsv_to_rgb(torch.stack([(hsv[..., 0] + delta) % 1.0, hsv[..., 1], hsv[..., 2]], -1))

    def adjust_saturation(x, scale, **kw):
        hsv = rgb_to_hsv(x)
        return hsv_to_rgb(torch.stack([hsv[..., 0], (hsv[..., 1] * scale).clamp(0, 1), hsv[..., 2]], -1))

    def nms_padded(boxes, scores, m, it, st, pad_to_max_output_size=False, **kw):
        sel = nms_v3(boxes, scores, m, it, st)
        n = torch.tensor(sel.numel(), dtype=torch.int32)
        if pad_to_max_output_size:
            sel = F.pad(sel, (0, int(m) - sel.numel()))
        return sel, n

    def nms_v5(boxes, scores, m, it, st, soft_nms_sigma=0.0, pad_to_max_output_size=False, **kw):
        if float(soft_nms_sigma) != 0.0:
            raise NotImplementedError("NonMaxSuppressionV5 with soft-NMS")
        sel, n = nms_padded(boxes, scores, m, it, st, pad_to_max_output_size)
        return sel, scores[sel.long()], n

    def unique(x, out_idx=None, **kw):
        seen, vals, idx = {}, [], []
        for v in x.tolist():
            if v not in seen:
                seen[v] = len(vals)
                vals.append(v)
            idx.append(seen[v])
        return torch.tensor(vals, dtype=x.dtype), torch.tensor(idx, dtype=torch.int32)

    def unique_counts(x, **kw):
        v, i = unique(x)
        return v, i, torch.bincount(i.long(), minlength=v.numel()).to(torch.int32)

    def list_diff(x, y, **kw):
        drop = set(y.tolist())
        keep = [j for j, v in enumerate(x.tolist()) if v not in drop]
        return x[keep], torch.tensor(keep, dtype=torch.int32)

    def polygamma(n, x, **kw):
        return torch.stack([torch.special.polygamma(int(k), v) for k, v in zip(n.reshape(-1).tolist(), x.reshape(-1))]).reshape(x.shape) if torch.is_tensor(n) and n.numel() > 1 \
            else torch.special.polygamma(int(n), x)

    def lu(x, **kw):
        LU, piv = torch.linalg.lu_factor(x)
        perm = torch.arange(x.shape[-1]).repeat(*x.shape[:-2], 1) if x.dim() > 2 else torch.arange(x.shape[-1])
        pv = (piv - 1).long()
        for i in range(pv.shape[-1]):                                                   # LAPACK row swaps -> permutation vector
            j = pv[..., i]
            a, b = perm[..., i].clone(), perm.gather(-1, j.unsqueeze(-1)).squeeze(-1)
            perm[..., i] = b
            perm.scatter_(-1, j.unsqueeze(-1), a.unsqueeze(-1))
        return LU, perm.to(torch.int32)

    def dilation2d(x, filt, strides=(1, 1, 1, 1), rates=(1, 1, 1, 1), padding="VALID", **kw):
        if s_(padding) != "VALID":
            raise NotImplementedError("Dilation2D with SAME padding")
        xn = x.permute(0, 3, 1, 2)
        n, c = xn.shape[:2]
        kh, kw_ = filt.shape[:2]
        cols = F.unfold(xn, (kh, kw_), dilation=list(rates[1:3]), stride=list(strides[1:3])).reshape(n, c, kh * kw_, -1)
        y = (cols + filt.permute(2, 0, 1).reshape(1, c, kh * kw_, 1)).amax(2)
        oh = (xn.shape[2] - (kh - 1) * rates[1] - 1) // strides[1] + 1
        return y.reshape(n, c, oh, -1).permute(0, 2, 3, 1)

    def draw_boxes(images, boxes, colors=None, **kw):
        out = images.clone()
        N, H, W, C = out.shape
        for n in range(N):
            for bi, b in enumerate(boxes[n]):
                y1, x1, y2, x2 = [float(v) for v in b]
                r1, r2 = int(round(y1 * (H - 1))), int(round(y2 * (H - 1)))
                c1, c2 = int(round(x1 * (W - 1))), int(round(x2 * (W - 1)))
                if r1 > r2 or c1 > c2 or r1 >= H or c1 >= W or r2 < 0 or c2 < 0:
                    continue
                col = colors[bi % colors.shape[0]][:C].to(out.dtype) if colors is not None and torch.is_tensor(colors) and colors.numel() else \
                    torch.tensor([1.0, 1.0, 0.0, 1.0][:C] if C > 1 else [1.0], dtype=out.dtype)
                r1c, r2c, c1c, c2c = max(r1, 0), min(r2, H - 1), max(c1, 0), min(c2, W - 1)
                if r1 >= 0: out[n, r1, c1c:c2c + 1] = col
                if r2 < H: out[n, r2, c1c:c2c + 1] = col
                if c1 >= 0: out[n, r1c:r2c + 1, c1] = col
                if c2 < W: out[n, r1c:r2c + 1, c2] = col
        return out

    def conv3d_backprop_input(sizes, w, dy, strides=(1, 1, 1, 1, 1), padding="VALID", dilations=(1, 1, 1, 1, 1), **kw):
        out = _ints(sizes)
        st, dl = list(strides[1:4]), list(dilations[1:4])
        g = dy.permute(0, 4, 1, 2, 3)
        wk = w.permute(4, 3, 0, 1, 2)                                                   # DHWIO -> OIDHW; conv_transpose wants [in=O, out=I, ...]
        pads, opad = [], []
        for d in range(3):
            eff = (wk.shape[2 + d] - 1) * dl[d] + 1
            total = max((g.shape[2 + d] - 1) * st[d] + eff - out[1 + d], 0) if s_(padding) == "SAME" else 0
            pads.append(total // 2)
            opad.append(out[1 + d] - ((g.shape[2 + d] - 1) * st[d] - 2 * (total // 2) + eff))
        y = F.conv_transpose3d(g, wk, None, st, pads, [max(o, 0) for o in opad], 1, dl)
        y = y[:, :, :out[1], :out[2], :out[3]]
        return y.permute(0, 2, 3, 4, 1)

    def conv2d_backprop_filter(x, sizes, dy, strides=(1, 1, 1, 1), padding="VALID", dilations=(1, 1, 1, 1), **kw):
        kh, kw_, ci, co = _ints(sizes)
        xn, g = x.permute(0, 3, 1, 2).float(), dy.permute(0, 3, 1, 2).float()
        st, dl = list(strides[1:3]), list(dilations[1:3])
        pad = [0, 0]
        if s_(padding) == "SAME":
            flat = []
            for d in (1, 0):
                total = max((g.shape[2 + d] - 1) * st[d] + ([kh, kw_][d] - 1) * dl[d] + 1 - xn.shape[2 + d], 0)
                flat += [total // 2, total - total // 2]
            xn = F.pad(xn, flat)
        gw = torch.nn.grad.conv2d_weight(xn, (co, ci, kh, kw_), g, st, pad, dl)
        return gw.permute(2, 3, 1, 0).to(x.dtype)

    M = {
        "Acosh": (lambda x, **k: x.acosh(), 1), "Asinh": (lambda x, **k: x.asinh(), 1), "Atanh": (lambda x, **k: x.atanh(), 1),
        "Erfc": (lambda x, **k: x.erfc(), 1), "Lgamma": (lambda x, **k: x.lgamma(), 1), "Digamma": (lambda x, **k: x.digamma(), 1),
        "Igamma": (lambda a, x, **k: torch.special.gammainc(a, x), 1), "Igammac": (lambda a, x, **k: torch.special.gammaincc(a, x), 1),
        "Polygamma": (polygamma, 1), "Zeta": (lambda x, q, **k: torch.special.zeta(x, q), 1),
        "Xdivy": (lambda x, y, **k: torch.where(x == 0, torch.zeros_like(x), x / y), 1), "Xlogy": (lambda x, y, **k: torch.special.xlogy(x, y), 1),
        "DivNoNan": (lambda x, y, **k: torch.where(y == 0, torch.zeros_like(x), x / y), 1),
        "TruncateMod": (lambda x, y, **k: torch.fmod(x, y), 1),
        "ApproximateEqual": (lambda x, y, tolerance=1e-5, **k: (x - y).abs() < tolerance, 1),
        "BitwiseAnd": (lambda x, y, **k: x & y, 1), "BitwiseOr": (lambda x, y, **k: x | y, 1), "BitwiseXor": (lambda x, y, **k: x ^ y, 1),
        "LeftShift": (lambda x, y, **k: x << y, 1), "RightShift": (lambda x, y, **k: x >> y, 1),
        "Bitcast": (lambda x, type=None, **k: x.view(type) if isinstance(type, torch.dtype) else x, 1),
        "CheckNumerics": (lambda x, **k: x, 1), "Empty": (lambda shape, dtype=None, init=False, **k: torch.zeros(_ints(shape)), 1),
        "BroadcastArgs": (lambda a, b, **k: torch.tensor(list(torch.broadcast_shapes(tuple(_ints(a)), tuple(_ints(b)))), dtype=torch.int32), 1),
        "Concat": (lambda axis, *xs, **k: torch.cat(xs, int(axis)), 1),
        "Cross": (lambda a, b, **k: torch.linalg.cross(a, b), 1),
        "Diag": (lambda x, **k: torch.diag(x.reshape(-1)).reshape(list(x.shape) * 2), 1),
        "DiagPart": (lambda x, **k: x.reshape(int(np.prod(x.shape[:x.dim() // 2])), -1).diagonal().reshape(x.shape[:x.dim() // 2]), 1),
        "MatrixSetDiag": (matrix_set_diag, 1), "MatrixSetDiagV3": (matrix_set_diag, 1),
        "MatrixDeterminant": (lambda x, **k: torch.linalg.det(x), 1), "MatrixInverse": (lambda x, adjoint=False, **k: torch.linalg.inv(x.mH if adjoint else x), 1),
        "LogMatrixDeterminant": (lambda x, **k: tuple(torch.linalg.slogdet(x)), 2),
        "Cholesky": (lambda x, **k: torch.linalg.cholesky(x), 1),
        "MatrixSolve": (lambda a, b, adjoint=False, **k: torch.linalg.solve(a.mH if adjoint else a, b), 1),
        "MatrixTriangularSolve": (lambda a, b, lower=True, adjoint=False, **k: torch.linalg.solve_triangular(a.mH if adjoint else a, b, upper=(not lower) != bool(adjoint)), 1),
        "Qr": (lambda x, full_matrices=False, **k: tuple(torch.linalg.qr(x, mode="complete" if full_matrices else "reduced")), 2),
        "Svd": (lambda x, compute_uv=True, full_matrices=False, **k: (lambda u, s, vh: (s, u, vh.mH))(*torch.linalg.svd(x, full_matrices=bool(full_matrices))), 3),
        "Lu": (lu, 2),
        "DynamicPartition": (dynamic_partition, -1), "DynamicStitch": (dynamic_stitch, 1), "ParallelDynamicStitch": (dynamic_stitch, 1),
        "FakeQuantWithMinMaxArgs": (lambda x, min=-6.0, max=6.0, **k: fake_quant(x, min, max, **k), 1),
        "FakeQuantWithMinMaxVars": (lambda x, lo, hi, **k: fake_quant(x, lo, hi, **k), 1),
        "FusedBatchNormV2": T["FusedBatchNorm"] if "FusedBatchNorm" in T else T.get("FusedBatchNormV3"),
        "HistogramFixedWidth": (lambda v, rng, nbins, **k: torch.bucketize(v.reshape(-1).float().clamp(float(rng[0]), float(rng[1])),
                                                                             torch.linspace(float(rng[0]), float(rng[1]), int(nbins) + 1)[1:-1], right=True)
                                .bincount(minlength=int(nbins)).to(torch.int32), 1),
        "Bincount": (lambda arr, size, weights, **k: (torch.bincount(arr.reshape(-1).long(), weights.reshape(-1) if weights.numel() else None, minlength=int(size))[:int(size)]), 1),
        "InTopK": (lambda p, t, k=1, **kw: in_top_k(p, t, k), 1), "InTopKV2": (in_top_k, 1),
        "InvertPermutation": (lambda x, **k: torch.argsort(x.long()).to(x.dtype), 1),
        "LinSpace": (lambda a, b, n, **k: torch.linspace(float(a), float(b), int(n), dtype=a.dtype if a.dtype.is_floating_point else torch.float32), 1),
        "ListDiff": (list_diff, 2),
        "MaxPoolV2": (lambda x, ksize, strides, **k: T["MaxPool"][0](x, ksize=_ints(ksize), strides=_ints(strides), **k), 1),
        "MaxPoolWithArgmax": (max_pool_argmax, 2),
        "Multinomial": (lambda logits, n, seed=0, seed2=0, **k: torch.multinomial(logits.float().softmax(-1), int(n), True), 1),
        "RandomStandardNormal": (lambda shape, **k: torch.randn(_ints(shape)), 1),
        "TruncatedNormal": (lambda shape, **k: torch.nn.init.trunc_normal_(torch.empty(_ints(shape)), 0.0, 1.0, -2.0, 2.0), 1),
        "RandomUniformInt": (lambda shape, lo, hi, **k: torch.randint(int(lo), int(hi), _ints(shape), dtype=lo.dtype), 1),
        "RandomGamma": (lambda shape, alpha, **k: torch.distributions.Gamma(alpha.float().expand(_ints(shape) + list(alpha.shape)), 1.0).sample(), 1),
        "RandomShuffle": (lambda x, **k: x[torch.randperm(x.shape[0])], 1),
        "NonMaxSuppression": (lambda b, s, m, iou_threshold=0.5, **k: nms_v3(b, s, m, iou_threshold, float("-inf")), 1),
        "NonMaxSuppressionV2": (lambda b, s, m, it, **k: nms_v3(b, s, m, it, float("-inf")), 1),
        "NonMaxSuppressionV4": (nms_padded, 2), "NonMaxSuppressionV5": (nms_v5, 3),
        "ResizeArea": (resize("area"), 1), "ResizeBicubic": (resize("bicubic"), 1), "CropAndResize": (crop_and_resize, 1),
        "ExtractImagePatches": (extract_patches, 1), "Dilation2D": (dilation2d, 1), "DrawBoundingBoxes": (draw_boxes, 1), "DrawBoundingBoxesV2": (draw_boxes, 1),
        "RGBToHSV": (rgb_to_hsv, 1), "HSVToRGB": (hsv_to_rgb, 1), "AdjustHue": (adjust_hue, 1), "AdjustSaturation": (adjust_saturation, 1),
        "AdjustContrastV2": (lambda x, f, **k: (x - x.mean((-3, -2), keepdim=True)) * f + x.mean((-3, -2), keepdim=True), 1),
        "Reverse": (lambda x, dims, **k: x.flip([i for i, d in enumerate(dims.tolist()) if d]) if dims.any() else x, 1),
        "ReverseSequence": (lambda x, lens, seq_dim=1, batch_dim=0, **k: torch.stack(
            [torch.cat([r.narrow(seq_dim - (seq_dim > batch_dim), 0, int(n)).flip(seq_dim - (seq_dim > batch_dim)),
                        r.narrow(seq_dim - (seq_dim > batch_dim), int(n), r.shape[seq_dim - (seq_dim > batch_dim)] - int(n))], seq_dim - (seq_dim > batch_dim))
             for r, n in zip(x.unbind(batch_dim), lens.tolist())], batch_dim), 1),
        "Roll": (lambda x, shift, axis, **k: torch.roll(x, _ints(shift) if shift.dim() else int(shift), _ints(axis) if axis.dim() else int(axis)), 1),
        "SegmentSum": (segment("sum"), 1), "SegmentMean": (segment("mean"), 1), "SegmentProd": (segment("prod"), 1),
        "SegmentMax": (lambda d, i, **k: segment("max")(d, i), 1), "SegmentMin": (lambda d, i, **k: segment("min")(d, i), 1),
        "UnsortedSegmentSum": (segment("sum"), 1), "UnsortedSegmentProd": (segment("prod"), 1),
        "UnsortedSegmentMax": (segment("max"), 1), "UnsortedSegmentMin": (segment("min"), 1),
        "TensorScatterAdd": (tensor_scatter("add"), 1), "TensorScatterSub": (tensor_scatter("sub"), 1), "TensorScatterUpdate": (tensor_scatter("update"), 1),
        "TopK": (lambda x, k=1, sorted=True, **kw: tuple(torch.topk(x, int(k), sorted=True)), 2),
        "Unique": (unique, 2), "UniqueWithCounts": (unique_counts, 3),
        "BatchNormWithGlobalNormalization": (lambda t, m, v, beta, gamma, variance_epsilon=1e-3, scale_after_normalization=True, **k:
                                             (t - m) * torch.rsqrt(v + variance_epsilon) * (gamma if scale_after_normalization else 1.0) + beta, 1),
        "Betainc": (lambda a, b, x, **k: torch.as_tensor(__import__("scipy.special").special.betainc(a.numpy(), b.numpy(), x.numpy())), 1),
        "ClipByNorm": (lambda x, c, **k: x * torch.clamp(c / x.norm().clamp(min=1e-30), max=1.0), 1),
        "NthElement": (lambda x, n, reverse=False, **k: (x.sort(-1, descending=bool(reverse)).values)[..., int(n)], 1),
        "Conv3DBackpropInputV2": (conv3d_backprop_input, 1), "Conv2DBackpropFilter": (conv2d_backprop_filter, 1),
    }
    return {k: v for k, v in M.items() if v is not None and k not in T}


def _register_tf_ops():
    from ..ops.registry import has, op
    if has("tf.Less"):
        return
    for name, (fn, n_out) in _tf_ops().items():
        op("tf." + name, n_out=n_out, group="tf_import")(fn)


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

    # ops with dedicated rules below (they map onto the framework's own ops so that its fusions and kernels apply)
    _DIRECT = {"Const", "Placeholder", "PlaceholderWithDefault", "MatMul", "BiasAdd", "Conv2D", "DepthwiseConv2dNative", "MaxPool", "AvgPool", "Reshape",
               "Softmax", "LogSoftmax", "Squeeze", "ExpandDims", "ConcatV2", "Transpose", "FusedBatchNorm", "FusedBatchNormV3", "Pad", "Cast", "LeakyRelu",
               "NoOp", "Shape", "Pack", "ArgMax"}
    # TensorFlow 1.x control flow: the same dataflow primitives the SameDiff executor runs (frames, dead branches)
    _CONTROL = {"Enter": "enter", "RefEnter": "enter", "Exit": "exit", "RefExit": "exit", "Switch": "switch", "RefSwitch": "switch",
                "Merge": "merge", "RefMerge": "merge", "NextIteration": "next_iteration", "RefNextIteration": "next_iteration", "LoopCond": "loop_cond"}
    # TensorArray ops -> the list ops of the framework
    _TENSOR_ARRAY = {"TensorArrayV3": "tensorarrayv3", "TensorArrayWriteV3": "tensorarraywritev3", "TensorArrayReadV3": "tensorarrayreadv3",
                     "TensorArrayGatherV3": "tensorarraygatherv3", "TensorArrayScatterV3": "tensorarrayscatterv3", "TensorArraySizeV3": "tensorarraysizev3",
                     "TensorArrayConcatV3": "tensorarrayconcatv3", "TensorArraySplitV3": "tensorarraysplitv3"}

    @classmethod
    def supportedOps(cls):
        from ..ops import registry
        ta = {k for k, v in cls._TENSOR_ARRAY.items() if registry.has(v)}
        return sorted(set(cls.UNARY) | set(cls.BINARY) | set(cls.REDUCE) | cls._DIRECT | set(cls._CONTROL) | ta | set(_tf_ops()))

    def runImport(self, path_or_bytes, dynamicVariables=None):
        _register_helpers()
        _register_tf_ops()
        from ..ops import registry
        if isinstance(path_or_bytes, (bytes, bytearray, memoryview)):
            data = path_or_bytes
        else:
            with open(path_or_bytes, "rb") as f:
                data = f.read()
        nodes = parse_graphdef(data)
        known = set(self.supportedOps())
        unsupported = sorted({n["op"] for n in nodes if n["op"] not in known})
        if unsupported:
            raise NotImplementedError(f"TensorFlow import: no mapping rule for op types {unsupported}")
        generic = _tf_ops()
        sd = SameDiff.create()
        vars_, consts, patches = {}, {}, []          # vars_: (node name, output index) -> SDVariable

        def put(name, out):
            outs = list(out) if isinstance(out, (list, tuple)) else [out]
            for k, v in enumerate(outs):
                vars_[(name, k)] = v

        def ref(s):
            nm, idx = _base(s)
            return vars_.get((nm, idx))

        def inp(n, i):
            v = ref(n["inputs"][i])
            if v is None:
                raise ValueError(f"TensorFlow import: input {n['inputs'][i]!r} of {n['name']} is produced later in the file and is not a loop back edge")
            return v

        def cval(n, i):
            nm, _ = _base(n["inputs"][i])
            if nm not in consts:
                raise ValueError(f"TensorFlow import: input {i} of {n['name']} ({n['op']}) must be a constant")
            return consts[nm]

        def plain(a):
            out = {}
            for k, v in a.items():
                if k in ("T", "Tidx", "Tshape", "Tparams", "Tindices", "Tperm", "Tpaddings", "TI", "Taxis", "Index", "out_type", "_output_shapes", "_class",
                         "Tlen", "Tmultiples", "Tlabels", "output_type", "N", "dtype", "element_shape", "clear_after_read", "dynamic_size",
                         "identical_element_shapes", "tensor_array_name", "parallel_iterations", "validate_indices", "use_cudnn_on_gpu",
                         "explicit_paddings", "U", "is_training", "exponential_avg_factor"):
                    continue
                if isinstance(v, tuple) or isinstance(v, torch.Tensor) or v is None:
                    continue
                out[k] = list(v) if isinstance(v, list) else v
            return out
        for n in nodes:
            op_, a, name = n["op"], n["attrs"], n["name"]
            data_in = [i for i in n["inputs"] if not i.startswith("^")]
            n = dict(n, inputs=data_in)
            if op_ == "NoOp":
                continue
            if op_ == "Const":
                t = a["value"]
                consts[name] = t
                put(name, sd.var(name, t.clone()) if (self.trainable and t.is_floating_point() and t.dim() >= 1) else sd.constant(name, t.clone()))
            elif op_ in ("Placeholder", "PlaceholderWithDefault"):
                dt = _TF_TO_DT.get(a.get("dtype", ("dtype", 1))[1], DataType.FLOAT)
                shp = a.get("shape", ("shape", None))[1]
                put(name, sd.placeHolder(name, dt, *(shp or [])))
            elif op_ in self._CONTROL:
                kind = self._CONTROL[op_]
                if kind == "enter":
                    put(name, sd._op("enter", [inp(n, 0)], name=name, frameName=a.get("frame_name", "frame"), isConstant=bool(a.get("is_constant", False))))
                elif kind == "merge":
                    have = [ref(i) for i in n["inputs"]]
                    first = next(v for v in have if v is not None)
                    m = sd._op("merge", [v if v is not None else first for v in have], name=name)
                    node = sd._producer[m.name]
                    for k, v in enumerate(have):
                        if v is None:
                            patches.append((node, k, n["inputs"][k]))           # the back edge: filled in once NextIteration exists
                    put(name, m)
                elif kind == "switch":
                    put(name, sd._op("switch", [inp(n, 0), inp(n, 1)], name=name))
                else:
                    put(name, sd._op(kind, [inp(n, 0)], name=name))
            elif op_ in self._TENSOR_ARRAY:
                target = self._TENSOR_ARRAY[op_]
                put(name, sd._op(target, [inp(n, i) for i in range(len(n["inputs"]))], name=name, n_out=registry.get(target).n_out))
            elif op_ in self.UNARY:
                put(name, sd._op(self.UNARY[op_], [inp(n, 0)], name=name))
            elif op_ in self.BINARY:
                put(name, sd._op(self.BINARY[op_], [inp(n, 0), inp(n, 1)], name=name))
            elif op_ in self.REDUCE and _base(n["inputs"][1])[0] in consts:
                ax = cval(n, 1).reshape(-1).tolist()
                put(name, sd._op(self.REDUCE[op_], [inp(n, 0)], name=name, dimensions=[int(v) for v in ax], keepDims=bool(a.get("keep_dims", False))))
            elif op_ == "MatMul":
                put(name, sd._op("matmul", [inp(n, 0), inp(n, 1)], name=name, transposeX=bool(a.get("transpose_a", False)), transposeY=bool(a.get("transpose_b", False))))
            elif op_ == "BiasAdd":
                put(name, sd._op("tf_bias_add", [inp(n, 0), inp(n, 1)], name=name, data_format=a.get("data_format", "NHWC")))
            elif op_ in ("Conv2D", "DepthwiseConv2dNative"):
                put(name, sd._op("tf_conv2d", [inp(n, 0), inp(n, 1)], name=name, strides=list(a.get("strides", [1, 1, 1, 1])), padding=a.get("padding", "SAME"),
                                 dilations=list(a.get("dilations", [1, 1, 1, 1])), data_format=a.get("data_format", "NHWC"), depthwise=op_ != "Conv2D"))
            elif op_ in ("MaxPool", "AvgPool"):
                put(name, sd._op("tf_pool", [inp(n, 0)], name=name, kind="max" if op_ == "MaxPool" else "avg", ksize=list(a["ksize"]), strides=list(a["strides"]),
                                 padding=a.get("padding", "VALID"), data_format=a.get("data_format", "NHWC")))
            elif op_ == "Reshape" and _base(n["inputs"][1])[0] in consts:
                put(name, sd._op("reshape", [inp(n, 0)], name=name, shape=[int(v) for v in cval(n, 1).reshape(-1).tolist()]))
            elif op_ == "Reshape":
                put(name, sd._op("reshape", [inp(n, 0), inp(n, 1)], name=name))
            elif op_ in ("Softmax", "LogSoftmax"):
                put(name, sd._op("softmax" if op_ == "Softmax" else "log_softmax", [inp(n, 0)], name=name, dimension=-1))
            elif op_ == "Squeeze":
                dims = a.get("squeeze_dims") or None
                put(name, sd._op("squeeze", [inp(n, 0)], name=name, dimensions=None if not dims else [int(v) for v in dims]))
            elif op_ == "ExpandDims":
                put(name, sd._op("expand_dims", [inp(n, 0)], name=name, axis=int(cval(n, 1))))
            elif op_ == "ConcatV2":
                put(name, sd._op("concat", [inp(n, i) for i in range(len(n["inputs"]) - 1)], name=name, concatDimension=int(cval(n, len(n["inputs"]) - 1))))
            elif op_ == "Pack":
                put(name, sd._op("stack", [inp(n, i) for i in range(len(n["inputs"]))], name=name, axis=int(a.get("axis", 0))))
            elif op_ == "Transpose":
                put(name, sd._op("permute", [inp(n, 0)], name=name, dimensions=[int(v) for v in cval(n, 1).tolist()]))
            elif op_ in ("FusedBatchNorm", "FusedBatchNormV3"):
                put(name, sd._op("tf_fused_batchnorm", [inp(n, i) for i in range(5)], name=name, epsilon=float(a.get("epsilon", 1e-3)), data_format=a.get("data_format", "NHWC")))
            elif op_ == "Pad":
                put(name, sd._op("pad", [inp(n, 0)], name=name, paddings=cval(n, 1).tolist(), mode="CONSTANT", constant=0.0))
            elif op_ == "Cast":
                put(name, sd._op("cast", [inp(n, 0)], name=name, dtype=int(_TF_TO_DT.get(a["DstT"][1], DataType.FLOAT))))
            elif op_ == "LeakyRelu":
                put(name, sd._op("leakyrelu", [inp(n, 0)], name=name, alpha=float(a.get("alpha", 0.2))))
            elif op_ == "Shape":
                put(name, sd._op("shape_of", [inp(n, 0)], name=name))
            elif op_ == "ArgMax":
                put(name, sd._op("argmax", [inp(n, 0)], name=name, dimensions=[int(cval(n, 1))]))
            elif op_ in self.REDUCE:              # reduction whose axes are computed in the graph
                fn = {"Mean": "mean", "Sum": "sum", "Max": "amax", "Min": "amin", "Prod": "prod"}[op_]
                if not registry.has("tf.Reduce" + fn):
                    def mk(fn=fn):
                        def f(x, axis, keep_dims=False, **kw):
                            ax = tuple(_ints(axis))
                            if fn == "prod":
                                for d in sorted((v % x.dim() for v in ax), reverse=True):
                                    x = x.prod(d, keepdim=bool(keep_dims))
                                return x
                            return getattr(x, fn)(ax, keepdim=bool(keep_dims))
                        return f
                    registry.op("tf.Reduce" + fn, group="tf_import")(mk())
                put(name, sd._op("tf.Reduce" + fn, [inp(n, 0), inp(n, 1)], name=name, keep_dims=bool(a.get("keep_dims", False))))
            else:
                fn, n_out = generic[op_]
                if n_out == -1:
                    n_out = int(a.get("num_split") or a.get("num") or len(n["inputs"]))
                put(name, sd._op("tf." + op_, [inp(n, i) for i in range(len(n["inputs"]))], name=name, n_out=n_out, **plain(a)))
        for node, k, src in patches:
            v = ref(src)
            if v is None:
                raise ValueError(f"TensorFlow import: merge input {src!r} is never produced")
            node.inputs[k] = v.name
        sd._exec_plan = None
        consumed = {_base(i)[0] for n in nodes for i in n["inputs"]}
        self.outputs = [n["name"] for n in nodes if n["name"] not in consumed and n["op"] not in ("Const", "Placeholder", "NoOp")]
        return sd


def importFrozenTF(path_or_bytes, trainable=False):
    return TensorflowFrameworkImporter(trainable).runImport(path_or_bytes)
