"""Shape / indexing ops (``headers/shape.h``, shape-related entries of ``headers/parity_ops.h`` and
``headers/transforms.h``): reshape, permute, concat/split/stack, gather/scatter families, slicing,
padding, tiling, space<->batch/depth, one-hot, sequence masks, dynamic partition/stitch."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..nd.dtype import DataType
from .registry import op


def _ints(v):
    if v is None:
        return None
    if isinstance(v, torch.Tensor):
        return [int(e) for e in v.reshape(-1).tolist()]
    if isinstance(v, (int, float)):
        return [int(v)]
    return [int(e) for e in v]


def _td(dtype, default=torch.float32):
    if dtype is None:
        return default
    if isinstance(dtype, torch.dtype):
        return dtype
    if isinstance(dtype, str):
        return DataType.from_name(dtype).to_torch()
    return DataType(dtype).to_torch()


@op("reshape")
def reshape(x, shape_t=None, shape=None, order="c", **kw):
    s = _ints(shape if shape is not None else shape_t)
    if s and s[0] in (-99, 99, 102) and len(s) > 1 and abs(s[0]) in (99, 102):   # legacy leading order char
        order, s = ("f" if abs(s[0]) == 102 else "c"), s[1:]
    if order == "f" and x.dim() > 1:
        flat = x.permute(*reversed(range(x.dim()))).reshape(-1)
        return flat.reshape(tuple(reversed(s))).permute(*reversed(range(len(s))))
    return x.reshape(s)


op("reshape_no_copy")(reshape)
op("reshapeas")(lambda x, y, **kw: x.reshape(y.shape))
op("permute")(lambda x, perm_t=None, dimensions=None, **kw: x.permute(*(_ints(dimensions if dimensions is not None else perm_t) or list(reversed(range(x.dim()))))))
op("transpose")(lambda x, perm_t=None, dimensions=None, **kw: x.permute(*(_ints(dimensions if dimensions is not None else perm_t) or list(reversed(range(x.dim()))))))
op("linear_copy")(lambda x, **kw: x.clone())
op("shape_of", differentiable=False)(lambda x, **kw: torch.tensor(list(x.shape), dtype=torch.int64, device=x.device))
op("shapes_of", n_out=-1, differentiable=False)(lambda *xs, **kw: tuple(torch.tensor(list(x.shape), dtype=torch.int64) for x in xs))
op("set_shape")(lambda x, shape, **kw: x.reshape(_ints(shape)))
op("size", differentiable=False)(lambda x, **kw: torch.tensor(x.numel(), dtype=torch.int64, device=x.device))
op("size_at", differentiable=False)(lambda x, dim=0, **kw: torch.tensor(x.shape[int(dim)], dtype=torch.int64, device=x.device))
op("rank", differentiable=False)(lambda x, **kw: torch.tensor(x.dim(), dtype=torch.int32, device=x.device))
op("order")(lambda x, order="c", **kw: x.contiguous())
op("flatten_2d")(lambda x, axis=1, **kw: x.reshape(int(torch.tensor(x.shape[:int(axis)]).prod()) if axis else 1, -1))
op("broadcast_to")(lambda x, shape, **kw: x.expand(*_ints(shape)))
def _tile_to_shape(x, shape=None, **kw):
    """``tile_to_shape``: repeat ``x`` along every axis until it has ``shape`` (each target extent a multiple of the source's;
    libnd4j/include/ops/declarable/generic/shape/tile_to_shape.cpp)."""
    tgt = _ints(shape)
    src = [1] * (len(tgt) - x.dim()) + list(x.shape)
    if any(t % s for t, s in zip(tgt, src)):
        raise ValueError(f"tile_to_shape: {tuple(x.shape)} does not tile to {tuple(tgt)}")
    return x.reshape(src).repeat(*[t // s for t, s in zip(tgt, src)])


op("tile_to_shape")(_tile_to_shape)
op("tile_to_shape_bp")(lambda x, g, **kw: g.sum_to_size(x.shape))
op("evaluate_reduction_shape", differentiable=False)(
    lambda shape, dims, keepDims=False, **kw: torch.tensor(
        [1 if i in [d % len(_ints(shape)) for d in _ints(dims)] else s for i, s in enumerate(_ints(shape))
         if keepDims or i not in [d % len(_ints(shape)) for d in _ints(dims)]], dtype=torch.int64))
op("create", differentiable=False)(lambda shape, dtype=None, order="c", init=True, **kw: torch.zeros(_ints(shape), dtype=_td(dtype)))
op("create_view")(lambda x, *idx, **kw: x)


@op("squeeze")
def squeeze(x, axis_t=None, dimensions=None, **kw):
    d = _ints(dimensions if dimensions is not None else axis_t)
    if not d:
        return x.squeeze()
    for dd in sorted([i % x.dim() for i in d], reverse=True):
        x = x.squeeze(dd)
    return x


@op("expand_dims")
def expand_dims(x, axis_t=None, axis=None, **kw):
    a = axis if axis is not None else axis_t
    a = _ints(a)[0]
    return x.unsqueeze(a if a >= 0 else a + x.dim() + 1)


@op("concat")
def concat(*xs, concatDimension=0, isDynamicAxis=False, **kw):
    xs = list(xs)
    if isDynamicAxis:
        concatDimension = int(xs.pop().reshape(-1)[0])
    return torch.cat(xs, dim=int(concatDimension))


@op("concat_bp", n_out=-1)
def concat_bp(*args, concatDimension=0, **kw):
    *xs, g = args
    return tuple(torch.split(g, [x.shape[int(concatDimension)] for x in xs], dim=int(concatDimension)))


@op("stack", "parallel_stack")
def stack(*xs, dimension=0, **kw):
    return torch.stack(xs, dim=int(dimension))


class _UnstackFn(torch.autograd.Function):
    """``unbind`` whose backward recognises gradients that already sit side by side in one buffer (the fused
    attention backward writes dq/dk/dv into a packed [.., 3, ..] tensor) and returns that buffer instead of
    re-assembling it with a concatenation copy."""

    @staticmethod
    def forward(ctx, x, dim):
        ctx.dim, ctx.shape = dim, x.shape
        return tuple(x.unbind(dim))

    @staticmethod
    def backward(ctx, *grads):
        dim, shape = ctx.dim, ctx.shape
        g0 = next((g for g in grads if g is not None), None)
        if g0 is not None and all(g is not None for g in grads):
            strides = list(torch.empty(shape, device="meta").stride())
            sub = strides[:dim] + strides[dim + 1:]
            st = g0.untyped_storage().data_ptr()
            base = g0.storage_offset()
            if all(g.untyped_storage().data_ptr() == st and list(g.stride()) == sub and g.dtype == g0.dtype
                   and g.storage_offset() == base + i * strides[dim] for i, g in enumerate(grads)):
                return torch.as_strided(g0, tuple(shape), strides, base), None
        zeros = [g if g is not None else torch.zeros_like(g0) for g in grads]
        return torch.stack(zeros, dim), None


def _unstack(x, dimension=0, num=None, **kw):
    d = int(dimension) % x.dim()
    if x.requires_grad and torch.is_grad_enabled():
        return _UnstackFn.apply(x, d)
    return tuple(torch.unbind(x, dim=d))


op("unstack", n_out=-1)(_unstack)
@op("tear", n_out=-1)
def tear(x, dimensions=(0,), **kw):
    """All sub-arrays that span ``dimensions`` (the tensors-along-dimension of ``tear.cpp``): for a [3, 4] array and dimension 1,
    three arrays of shape [4]."""
    dims = sorted(d % x.dim() for d in _ints(dimensions))
    rest = [d for d in range(x.dim()) if d not in dims]
    y = x.permute(*rest, *dims).reshape(-1, *[x.shape[d] for d in dims])
    return tuple(y.unbind(0))


@op("split", n_out=-1)
def split(*args, numSplit=2, dimension=0, **kw):
    if len(args) == 2:   # (axis tensor, x) TF ordering
        a, x = args
        if a.numel() == 1 and a.dtype in (torch.int32, torch.int64) and x.dim() > 0:
            dimension = int(a)
        else:
            x, dimension = a, int(x)
    else:
        x = args[0]
    return tuple(torch.chunk(x, int(numSplit), dim=int(dimension)))


@op("split_v", n_out=-1)
def split_v(x, sizes, dimension=0, **kw):
    s = _ints(sizes)
    d = int(dimension)
    if -1 in s:
        s[s.index(-1)] = x.shape[d] - (sum(s) + 1)
    return tuple(torch.split(x, s, dim=d))


@op("slice")
def slice_(x, begin_t=None, size_t=None, begin=None, size=None, **kw):
    b = _ints(begin if begin is not None else begin_t)
    s = _ints(size if size is not None else size_t)
    idx = tuple(slice(bb, None if ss == -1 else bb + ss) for bb, ss in zip(b, s))
    return x[idx]


@op("slice_bp")
def slice_bp(x, *rest, begin=None, size=None, **kw):
    g = rest[-1]
    b = _ints(begin if begin is not None else rest[0])
    out = torch.zeros_like(x)
    idx = tuple(slice(bb, bb + gs) for bb, gs in zip(b, g.shape))
    out[idx] = g
    return out


def _strided_index(x, begin, end, strides, begin_mask=0, end_mask=0, ellipsis_mask=0, new_axis_mask=0, shrink_axis_mask=0):
    idx = []
    for i, (b, e, s) in enumerate(zip(begin, end, strides)):
        if ellipsis_mask & (1 << i):
            idx.append(Ellipsis)
            continue
        if new_axis_mask & (1 << i):
            idx.append(None)
            continue
        if shrink_axis_mask & (1 << i):
            idx.append(b)
            continue
        bb = None if begin_mask & (1 << i) else b
        ee = None if end_mask & (1 << i) else e
        idx.append(slice(bb, ee, s))
    return tuple(idx)


@op("strided_slice")
def strided_slice(x, begin_t=None, end_t=None, strides_t=None, begin=None, end=None, strides=None, begin_mask=0, end_mask=0,
                  ellipsis_mask=0, new_axis_mask=0, shrink_axis_mask=0, **kw):
    b = _ints(begin if begin is not None else begin_t)
    e = _ints(end if end is not None else end_t)
    s = _ints(strides if strides is not None else strides_t) or [1] * len(b)
    idx = _strided_index(x, b, e, s, begin_mask, end_mask, ellipsis_mask, new_axis_mask, shrink_axis_mask)
    if any(isinstance(i, slice) and i.step is not None and i.step < 0 for i in idx):
        # negative strides: flip then slice
        out = x
        new = []
        for d, i in enumerate(idx):
            if isinstance(i, slice) and i.step is not None and i.step < 0:
                n = x.shape[d]
                start = n - 1 if i.start is None else (i.start if i.start >= 0 else n + i.start)
                stop = -1 if i.stop is None else (i.stop if i.stop >= 0 else n + i.stop)
                out = out.flip(d)
                new.append(slice(n - 1 - start, n - 1 - stop, -i.step))
            else:
                new.append(i)
        return out[tuple(new)]
    return x[idx]


@op("strided_slice_bp")
def strided_slice_bp(x, *rest, **kw):
    g = rest[-1]
    xx = x.detach().requires_grad_(True)
    with torch.enable_grad():
        y = strided_slice(xx, *rest[:-1], **kw)
    return torch.autograd.grad(y, xx, g.reshape(y.shape))[0]


@op("gather")
def gather(x, indices=None, axis=0, intArgs=None, **kw):
    idx = indices if indices is not None else torch.tensor(intArgs, device=x.device)
    if isinstance(axis, torch.Tensor):
        axis = int(axis)
    if int(axis) == 0 and x.dim() == 2 and x.is_cuda:
        from . import native as nat
        y = nat.gather_rows(x, idx)          # gradient scattered in fp32, straight into the table's master gradient
        if y is not None:
            return y.reshape(tuple(idx.shape) + x.shape[1:])
    return torch.index_select(x, int(axis), idx.reshape(-1).long()).reshape(
        x.shape[:int(axis)] + tuple(idx.shape) + x.shape[int(axis) + 1:])


op("embedding_lookup")(lambda x, idx, partition_mode=0, **kw: x[idx.long()])


@op("gather_nd")
def gather_nd(x, indices, checkIndices=False, **kw):
    idx = indices.long()
    return x[tuple(idx[..., i] for i in range(idx.shape[-1]))]


def _scatter(mode):
    def run(x, indices, updates, lock=False, checkIndices=False, **kw):
        out = x.clone()
        idx = indices.long()
        if idx.dim() == 0:
            idx = idx.reshape(1)
            updates = updates.unsqueeze(0)
        flat_idx = idx.reshape(-1)
        upd = updates.reshape((flat_idx.numel(),) + tuple(x.shape[1:]))
        if mode == "upd":
            out[flat_idx] = upd.to(out.dtype)
            return out
        ii = flat_idx.reshape([-1] + [1] * (x.dim() - 1)).expand_as(upd)
        if mode == "add":
            return out.scatter_add(0, ii, upd.to(out.dtype))
        if mode == "sub":
            return out.scatter_add(0, ii, -upd.to(out.dtype))
        red = {"mul": "prod", "max": "amax", "min": "amin"}.get(mode)
        if mode == "div":
            return out.scatter_reduce(0, ii, 1.0 / upd.to(out.dtype), "prod", include_self=True)
        return out.scatter_reduce(0, ii, upd.to(out.dtype), red, include_self=True)
    return run


for _m in ("add", "sub", "mul", "div", "upd", "max", "min"):
    op(f"scatter_{_m}")(_scatter(_m))


@op("scatter_update")
def scatter_update(x, updates, opCode=0, dimensions=None, indices=None, **kw):
    mode = ["add", "sub", "mul", "div", "rsub", "rdiv", "upd"][int(opCode)]
    idx = torch.as_tensor(indices, device=x.device)
    return _scatter(mode if mode in ("add", "sub", "mul", "div", "upd") else "upd")(x, idx, updates)


@op("scatter_nd")
def scatter_nd(indices, updates, shape, **kw):
    out = torch.zeros(_ints(shape), dtype=updates.dtype, device=updates.device)
    return scatter_nd_add(out, indices, updates)


@op("scatter_nd_add")
def scatter_nd_add(x, indices, updates, **kw):
    idx = indices.long()
    return x.index_put(tuple(idx[..., i] for i in range(idx.shape[-1])), updates.to(x.dtype), accumulate=True)


op("scatter_nd_sub")(lambda x, indices, updates, **kw: scatter_nd_add(x, indices, -updates))


@op("scatter_nd_update")
def scatter_nd_update(x, indices, updates, **kw):
    idx = indices.long()
    return x.index_put(tuple(idx[..., i] for i in range(idx.shape[-1])), updates.to(x.dtype), accumulate=False)


@op("tile")
def tile(x, reps_t=None, reps=None, **kw):
    r = _ints(reps if reps is not None else reps_t)
    return x.repeat(*r)


op("tile_bp")(lambda x, *rest, **kw: rest[-1].reshape(
    [v for pair in zip([s // o for s, o in zip(rest[-1].shape, x.shape)], x.shape) for v in pair]).sum(
    dim=list(range(0, 2 * x.dim(), 2))))
op("repeat")(lambda x, repeats=None, dimension=0, **kw: torch.repeat_interleave(
    x, torch.as_tensor(_ints(repeats), device=x.device) if len(_ints(repeats)) > 1 else _ints(repeats)[0], dim=int(dimension)))


@op("pad")
def pad(x, paddings, mode=0, padValue=0.0, **kw):
    p = paddings.long().reshape(-1, 2).tolist() if isinstance(paddings, torch.Tensor) else [list(q) for q in paddings]
    flat = []
    for lo, hi in reversed(p):
        flat += [int(lo), int(hi)]
    m = {0: "constant", 1: "reflect", 2: "symmetric"}.get(int(mode), "constant")
    if m == "constant":
        return F.pad(x, flat, value=float(padValue))
    return mirror_pad(x, paddings, isSymmetric=(m == "symmetric"))


@op("mirror_pad")
def mirror_pad(x, paddings, isSymmetric=False, mode=None, **kw):
    if mode is not None:
        isSymmetric = int(mode) == 1
    p = paddings.long().reshape(-1, 2).tolist() if isinstance(paddings, torch.Tensor) else [list(q) for q in paddings]
    out = x
    for d, (lo, hi) in enumerate(p):
        n = out.shape[d]
        off = 0 if isSymmetric else 1
        pieces = []
        if lo:
            pieces.append(out.narrow(d, off, lo).flip(d))
        pieces.append(out)
        if hi:
            pieces.append(out.narrow(d, n - hi - off, hi).flip(d))
        out = torch.cat(pieces, d)
    return out


op("reverse")(lambda x, dims_t=None, dimensions=None, **kw: x.flip(*[d % x.dim() for d in (_ints(dimensions if dimensions is not None else dims_t) or range(x.dim()))]))
op("reverse_bp")(lambda x, *rest, dimensions=None, **kw: rest[-1].flip(*[d % x.dim() for d in (_ints(dimensions) or range(x.dim()))]))


@op("reverse_sequence")
def reverse_sequence(x, seqLengths, seqDim=1, batchDim=0, **kw):
    out = x.clone()
    for b in range(x.shape[int(batchDim)]):
        n = int(seqLengths[b])
        sl = out.select(int(batchDim), b)
        d = int(seqDim) - (1 if int(seqDim) > int(batchDim) else 0)
        sl.narrow(d, 0, n).copy_(x.select(int(batchDim), b).narrow(d, 0, n).flip(d))
    return out


@op("roll")
def roll(x, shift_t=None, dims_t=None, shift=None, dimensions=None, **kw):
    s = _ints(shift if shift is not None else shift_t)
    d = _ints(dimensions if dimensions is not None else dims_t)
    if not d:
        return torch.roll(x.reshape(-1), s[0]).reshape(x.shape)
    return torch.roll(x, s if len(s) == len(d) else s * len(d), d)


@op("onehot", "one_hot")
def onehot(idx, depth=None, on=1.0, off=0.0, axis=-1, dtype=None, **kw):
    depth = int(depth)
    oh = F.one_hot(idx.long().clamp(0, depth - 1), depth).to(_td(dtype))
    oh = oh * (on - off) + off
    valid = ((idx >= 0) & (idx < depth)).unsqueeze(-1)
    oh = torch.where(valid, oh, torch.full_like(oh, off))
    axis = int(axis)
    return oh if axis in (-1, idx.dim()) else oh.movedim(-1, axis)


@op("sequence_mask", differentiable=False)
def sequence_mask(lengths, maxLen=None, dtype=None, **kw):
    m = int(maxLen) if maxLen is not None and not isinstance(maxLen, torch.Tensor) else (int(maxLen) if maxLen is not None else int(lengths.max()))
    r = torch.arange(m, device=lengths.device)
    return (r < lengths.unsqueeze(-1)).to(_td(dtype, torch.bool))


op("range", differentiable=False)(lambda *a, frm=0, to=None, step=1, dtype=None, **kw: torch.arange(
    *( [float(v) if isinstance(v, torch.Tensor) and v.dtype.is_floating_point else (int(v) if isinstance(v, torch.Tensor) else v) for v in a]
       if a else [frm, to, step]), dtype=_td(dtype, None) if dtype is not None else None))
op("lin_space", "linspace", differentiable=False)(lambda *a, start=0.0, stop=1.0, number=2, dtype=None, **kw: torch.linspace(
    float(a[0]) if a else start, float(a[1]) if len(a) > 1 else stop, int(a[2]) if len(a) > 2 else int(number), dtype=_td(dtype)))
op("eye", differentiable=False)(lambda *a, rows=None, cols=None, dtype=None, **kw: torch.eye(
    int(a[0]) if a else int(rows), int(a[1]) if len(a) > 1 else int(cols if cols is not None else (a[0] if a else rows)), dtype=_td(dtype)))
op("fill", differentiable=False)(lambda shape, value=0.0, dtype=None, **kw: torch.full(_ints(shape), float(value), dtype=_td(dtype)))
op("fill_as")(lambda x, value=0.0, **kw: torch.full_like(x, float(value)))
op("tri", differentiable=False)(lambda rows=1, cols=None, diag=0, dtype=None, **kw: torch.tril(torch.ones(int(rows), int(cols or rows), dtype=_td(dtype)), int(diag)))
op("triu")(lambda x, diag=0, **kw: torch.triu(x, int(diag)))
op("triu_bp")(lambda x, g, diag=0, **kw: torch.triu(g, int(diag)))
op("matrix_band_part")(lambda x, minLower=-1, maxUpper=-1, **kw: _band(x, int(minLower), int(maxUpper)))


def _band(x, lo, hi):
    m, n = x.shape[-2:]
    i = torch.arange(m, device=x.device).unsqueeze(1)
    j = torch.arange(n, device=x.device).unsqueeze(0)
    keep = ((lo < 0) | (i - j <= lo)) & ((hi < 0) | (j - i <= hi))
    return x * keep.to(x.dtype)


op("diag")(lambda x, **kw: torch.diag_embed(x.reshape(-1)).reshape(tuple(x.shape) * 2))
op("diag_part")(lambda x, **kw: x.reshape(int(x.numel() ** 0.5), -1).diagonal().reshape(x.shape[:x.dim() // 2]))
op("matrix_diag")(lambda x, **kw: torch.diag_embed(x))
op("matrix_diag_part")(lambda x, **kw: torch.diagonal(x, dim1=-2, dim2=-1))
op("matrix_set_diag")(lambda x, d, **kw: x - torch.diag_embed(torch.diagonal(x, dim1=-2, dim2=-1)) + torch.diag_embed(d))
op("trace")(lambda x, **kw: torch.diagonal(x, dim1=-2, dim2=-1).sum(-1))
op("invert_permutation", differentiable=False)(lambda x, **kw: torch.argsort(x))
op("meshgrid", n_out=-1)(lambda *xs, cartesian=True, **kw: tuple(torch.meshgrid(*xs, indexing="xy" if cartesian else "ij")))
op("broadcast_dynamic_shape", differentiable=False)(
    lambda a, b, **kw: torch.tensor(list(torch.broadcast_shapes(tuple(_ints(a)), tuple(_ints(b)))), dtype=torch.int64))
op("broadcastgradientargs", n_out=2, differentiable=False)(lambda a, b, **kw: _bga(_ints(a), _ints(b)))


def _bga(a, b):
    n = max(len(a), len(b))
    pa, pb = [1] * (n - len(a)) + a, [1] * (n - len(b)) + b
    ra = [i for i in range(n) if pa[i] == 1 and pb[i] != 1]
    rb = [i for i in range(n) if pb[i] == 1 and pa[i] != 1]
    return torch.tensor(ra, dtype=torch.int64), torch.tensor(rb, dtype=torch.int64)


@op("space_to_depth")
def space_to_depth(x, blockSize=2, isNHWC=False, **kw):
    b = int(blockSize)
    if isNHWC:
        x = x.permute(0, 3, 1, 2)
    n, c, h, w = x.shape
    y = x.reshape(n, c, h // b, b, w // b, b).permute(0, 3, 5, 1, 2, 4).reshape(n, c * b * b, h // b, w // b)
    return y.permute(0, 2, 3, 1) if isNHWC else y


@op("depth_to_space")
def depth_to_space(x, blockSize=2, isNHWC=False, **kw):
    b = int(blockSize)
    if isNHWC:
        x = x.permute(0, 3, 1, 2)
    n, c, h, w = x.shape
    y = x.reshape(n, b, b, c // (b * b), h, w).permute(0, 3, 4, 1, 5, 2).reshape(n, c // (b * b), h * b, w * b)
    return y.permute(0, 2, 3, 1) if isNHWC else y


@op("space_to_batch", "space_to_batch_nd")
def space_to_batch(x, *rest, blockSize=2, blocks=None, padding=None, **kw):
    # NHWC layout, as in TF
    if rest and blocks is None and len(rest) == 2:
        blocks, padding = _ints(rest[0]), rest[1].long().reshape(-1, 2).tolist()
    elif rest:
        padding = rest[0].long().reshape(-1, 2).tolist()
    blocks = blocks or [int(blockSize)] * 2
    p = padding or [[0, 0], [0, 0]]
    x = F.pad(x, [0, 0, p[1][0], p[1][1], p[0][0], p[0][1]])
    n, h, w, c = x.shape
    bh, bw = blocks
    y = x.reshape(n, h // bh, bh, w // bw, bw, c).permute(2, 4, 0, 1, 3, 5)
    return y.reshape(n * bh * bw, h // bh, w // bw, c)


@op("batch_to_space", "batch_to_space_nd")
def batch_to_space(x, *rest, blockSize=2, blocks=None, crops=None, **kw):
    if rest and blocks is None and len(rest) == 2:
        blocks, crops = _ints(rest[0]), rest[1].long().reshape(-1, 2).tolist()
    elif rest:
        crops = rest[0].long().reshape(-1, 2).tolist()
    blocks = blocks or [int(blockSize)] * 2
    c_ = crops or [[0, 0], [0, 0]]
    bh, bw = blocks
    nb, h, w, c = x.shape
    n = nb // (bh * bw)
    y = x.reshape(bh, bw, n, h, w, c).permute(2, 3, 0, 4, 1, 5).reshape(n, h * bh, w * bw, c)
    return y[:, c_[0][0]:y.shape[1] - c_[0][1], c_[1][0]:y.shape[2] - c_[1][1], :]


@op("dynamic_partition", n_out=-1, differentiable=False)
def dynamic_partition(x, partitions, numPartitions=2, **kw):
    return tuple(x[partitions == i] for i in range(int(numPartitions)))


@op("dynamic_partition_bp", n_out=-1)
def dynamic_partition_bp(x, partitions, *grads, numPartitions=2, **kw):
    out = torch.zeros_like(x)
    for i, g in enumerate(grads):
        out[partitions == i] = g
    return out, torch.zeros_like(partitions)


@op("dynamic_stitch")
def dynamic_stitch(*args, numPartitions=None, **kw):
    n = len(args) // 2
    idx, data = args[:n], args[n:]
    size = max(int(i.max()) for i in idx if i.numel()) + 1
    out = torch.zeros((size,) + tuple(data[0].shape[idx[0].dim():]), dtype=data[0].dtype, device=data[0].device)
    for i, d in zip(idx, data):
        out[i.reshape(-1).long()] = d.reshape((-1,) + tuple(out.shape[1:]))
    return out


op("flatten")(lambda *xs, order="c", **kw: torch.cat([
    (x.permute(*reversed(range(x.dim()))) if order == "f" and x.dim() > 1 else x).reshape(-1) for x in xs]))
op("stop_gradient")(lambda x, **kw: x.detach())
op("noop", n_out=-1)(lambda *xs, **kw: tuple(xs))
op("merge")(lambda *xs, **kw: next(x for x in xs if x is not None))
op("cross")(lambda a, b, **kw: torch.linalg.cross(a, b, dim=-1))


@op("compare_and_bitpack", differentiable=False)
def compare_and_bitpack(x, threshold, **kw):
    bits = (x > threshold).to(torch.uint8).reshape(-1, 8)
    w = torch.tensor([128, 64, 32, 16, 8, 4, 2, 1], dtype=torch.uint8, device=x.device)
    return (bits * w).sum(1).to(torch.uint8).reshape(x.shape[:-1] + (x.shape[-1] // 8,))


@op("extract_image_patches")
def extract_image_patches(x, kH=1, kW=1, sH=1, sW=1, rH=1, rW=1, isSameMode=False, **kw):
    # NHWC in/out
    xc = x.permute(0, 3, 1, 2)
    if isSameMode:
        oh, ow = -(-xc.shape[2] // sH), -(-xc.shape[3] // sW)
        ph = max((oh - 1) * sH + (kH - 1) * rH + 1 - xc.shape[2], 0)
        pw = max((ow - 1) * sW + (kW - 1) * rW + 1 - xc.shape[3], 0)
        xc = F.pad(xc, [pw // 2, pw - pw // 2, ph // 2, ph - ph // 2])
    cols = F.unfold(xc, (kH, kW), dilation=(rH, rW), stride=(sH, sW))
    n, c = xc.shape[:2]
    oh = (xc.shape[2] - (kH - 1) * rH - 1) // sH + 1
    ow = (xc.shape[3] - (kW - 1) * rW - 1) // sW + 1
    return cols.reshape(n, c, kH * kW, oh, ow).permute(0, 3, 4, 2, 1).reshape(n, oh, ow, kH * kW * c)
