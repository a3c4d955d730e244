"""Reductions: ``reduce_*`` custom ops (+ ``_bp``), legacy reduce / reduce3 / index-reduce /
summary-stats families (``libnd4j/include/loops/legacy_ops.h:96-131``), cumulative ops, moments,
segment reductions (``helpers/cuda/segment*.cu``) and top-k style selections."""
from __future__ import annotations

import torch

from .registry import op


def _dims(x, dimensions):
    if dimensions is None or (isinstance(dimensions, (list, tuple)) and len(dimensions) == 0):
        return None
    if isinstance(dimensions, torch.Tensor):
        dimensions = dimensions.reshape(-1).tolist()
    if isinstance(dimensions, int):
        dimensions = [dimensions]
    return tuple(int(d) % max(x.dim(), 1) for d in dimensions)


def _reduce(fn):
    def run(x, dimensions=None, keepDims=False, **kw):
        d = _dims(x, dimensions)
        if d is None:
            r = fn(x, tuple(range(x.dim())), False)
            return r.reshape([1] * x.dim()) if keepDims else r
        return fn(x, d, keepDims)
    return run


def _reg(name, fn, *aliases, bp=True, differentiable=True):
    run = _reduce(fn)
    op(name, *aliases, differentiable=differentiable)(run)
    if bp:
        @op(name + "_bp")
        def _b(x, g, dimensions=None, keepDims=False, **kw):
            x = x.detach().requires_grad_(True)
            with torch.enable_grad():
                y = run(x, dimensions, keepDims)
            return torch.autograd.grad(y, x, g.reshape(y.shape).to(y.dtype))[0]


def _prod(x, d, k):
    for dd in sorted(d, reverse=True):
        x = x.prod(dim=dd, keepdim=True)
    return x if k else x.reshape([s for i, s in enumerate(x.shape) if i not in d])


_reg("reduce_sum", lambda x, d, k: x.sum(d, keepdim=k), "sum")
_reg("reduce_mean", lambda x, d, k: x.mean(d, keepdim=k), "mean")
_reg("reduce_prod", _prod, "prod")
_reg("reduce_max", lambda x, d, k: x.amax(d, keepdim=k), "max")
_reg("reduce_min", lambda x, d, k: x.amin(d, keepdim=k), "min")
_reg("reduce_norm1", lambda x, d, k: x.abs().sum(d, keepdim=k), "norm1")
_reg("reduce_norm2", lambda x, d, k: (x * x).sum(d, keepdim=k).sqrt(), "norm2")
_reg("reduce_sqnorm", lambda x, d, k: (x * x).sum(d, keepdim=k), "squarednorm")
_reg("reduce_norm_max", lambda x, d, k: x.abs().amax(d, keepdim=k), "normmax")
_reg("reduce_logsumexp", lambda x, d, k: torch.logsumexp(x, d, keepdim=k), "logsumexp", bp=False)
_reg("amax", lambda x, d, k: x.abs().amax(d, keepdim=k), bp=False)
_reg("amin", lambda x, d, k: x.abs().amin(d, keepdim=k), bp=False)
_reg("amean", lambda x, d, k: x.abs().mean(d, keepdim=k), bp=False)
_reg("asum", lambda x, d, k: x.abs().sum(d, keepdim=k), bp=False)
_reg("entropy", lambda x, d, k: -(x * x.log()).sum(d, keepdim=k), bp=False)
_reg("log_entropy", lambda x, d, k: (-(x * x.log()).sum(d, keepdim=k)).log(), bp=False)
_reg("shannonentropy", lambda x, d, k: -(x * x.log2()).sum(d, keepdim=k), bp=False)
_reg("countNonZero", lambda x, d, k: (x != 0).sum(d, keepdim=k), "count_non_zero", bp=False, differentiable=False)
_reg("countZero", lambda x, d, k: (x == 0).sum(d, keepdim=k), "count_zero", bp=False, differentiable=False)
_reg("any", lambda x, d, k: (x != 0).any(dim=d[0], keepdim=k) if len(d) == 1 else (x != 0).sum(d, keepdim=k) > 0, bp=False, differentiable=False)
_reg("all", lambda x, d, k: (x != 0).all(dim=d[0], keepdim=k) if len(d) == 1 else (x == 0).sum(d, keepdim=k) == 0, bp=False, differentiable=False)
_reg("isnan_any", lambda x, d, k: torch.isnan(x).sum(d, keepdim=k) > 0, bp=False, differentiable=False)
_reg("isinf_any", lambda x, d, k: torch.isinf(x).sum(d, keepdim=k) > 0, bp=False, differentiable=False)


@op("reduce_variance", "variance", "var")
def reduce_variance(x, dimensions=None, keepDims=False, biasCorrected=False, **kw):
    d = _dims(x, dimensions)
    return x.var(dim=d, unbiased=bool(biasCorrected), keepdim=keepDims)


@op("reduce_stdev", "standarddeviation", "std")
def reduce_stdev(x, dimensions=None, keepDims=False, biasCorrected=False, **kw):
    d = _dims(x, dimensions)
    return x.std(dim=d, unbiased=bool(biasCorrected), keepdim=keepDims)


for _n, _f in (("reduce_variance_bp", reduce_variance), ("reduce_stdev_bp", reduce_stdev)):
    def _mk(_f):
        def run(x, g, dimensions=None, keepDims=False, biasCorrected=False, **kw):
            x = x.detach().requires_grad_(True)
            with torch.enable_grad():
                y = _f(x, dimensions, keepDims, biasCorrected)
            return torch.autograd.grad(y, x, g.reshape(y.shape))[0]
        return run
    op(_n)(_mk(_f))


@op("reduce_dot_bp", n_out=2)
def reduce_dot_bp(x, y, g, dimensions=None, keepDims=False, **kw):
    d = _dims(x, dimensions)
    gg = g
    if d is not None and not keepDims:
        for dd in sorted(d):
            gg = gg.unsqueeze(dd)
    return gg * y, gg * x


@op("moments", n_out=2)
def moments(x, dimensions=None, keepDims=False, **kw):
    d = _dims(x, dimensions)
    return x.mean(dim=d, keepdim=keepDims), x.var(dim=d, unbiased=False, keepdim=keepDims)


@op("normalize_moments", n_out=2)
def normalize_moments(counts, means, variances, shift=0.0, **kw):
    m = means / counts + shift
    return m, variances / counts - (means / counts) ** 2


@op("sufficient_statistics", n_out=-1)
def sufficient_statistics(x, dimensions, shift=None, **kw):
    d = _dims(x, dimensions)
    cnt = torch.tensor(float(torch.tensor([x.shape[i] for i in d]).prod()), dtype=x.dtype, device=x.device)
    xs = x - shift if shift is not None else x
    out = (cnt, xs.sum(d), (xs * xs).sum(d))
    return out + ((shift,) if shift is not None else ())


# ----------------------------------------------------------------------------- reduce3 (pairwise distances)
def _r3(name, fn, *aliases):
    @op(name, *aliases)
    def run(x, y, dimensions=None, keepDims=False, **kw):
        d = _dims(x, dimensions)
        d = d if d is not None else tuple(range(x.dim()))
        return fn(x, y, d, keepDims)


_r3("dot", lambda x, y, d, k: (x * y).sum(d, keepdim=k))
_r3("cosinesimilarity", lambda x, y, d, k: (x * y).sum(d, keepdim=k) / ((x * x).sum(d, keepdim=k).sqrt() * (y * y).sum(d, keepdim=k).sqrt()))
_r3("cosinedistance", lambda x, y, d, k: 1 - (x * y).sum(d, keepdim=k) / ((x * x).sum(d, keepdim=k).sqrt() * (y * y).sum(d, keepdim=k).sqrt()))
_r3("euclidean", lambda x, y, d, k: ((x - y) ** 2).sum(d, keepdim=k).sqrt(), "euclideandistance")
_r3("manhattan", lambda x, y, d, k: (x - y).abs().sum(d, keepdim=k), "manhattandistance")
_r3("hammingdistance", lambda x, y, d, k: (x != y).to(x.dtype).sum(d, keepdim=k))
_r3("jaccarddistance", lambda x, y, d, k: 1 - torch.minimum(x, y).sum(d, keepdim=k) / torch.maximum(x, y).sum(d, keepdim=k))
_r3("equals_with_eps", lambda x, y, d, k: ((x - y).abs() > 1e-5).sum(d, keepdim=k))


# ----------------------------------------------------------------------------- index reductions
def _idx(name, fn, *aliases):
    @op(name, *aliases, differentiable=False)
    def run(x, dimensions=None, keepDims=False, **kw):
        d = _dims(x, dimensions)
        if d is None:
            return fn(x.reshape(-1), 0, False)
        if len(d) == 1:
            return fn(x, d[0], keepDims)
        other = [i for i in range(x.dim()) if i not in d]
        xp = x.permute(*other, *d).reshape([x.shape[i] for i in other] + [-1])
        return fn(xp, -1, keepDims)


_idx("argmax", lambda x, d, k: x.argmax(dim=d, keepdim=k), "imax")
_idx("argmin", lambda x, d, k: x.argmin(dim=d, keepdim=k), "imin")
_idx("argamax", lambda x, d, k: x.abs().argmax(dim=d, keepdim=k), "iamax")
_idx("argamin", lambda x, d, k: x.abs().argmin(dim=d, keepdim=k), "iamin")
_idx("firstindex", lambda x, d, k: (x != 0).to(torch.int64).argmax(dim=d, keepdim=k))
_idx("lastindex", lambda x, d, k: x.shape[d] - 1 - (x != 0).flip(d).to(torch.int64).argmax(dim=d, keepdim=k))


@op("norm")
def norm(x, mode=2, dimensions=None, **kw):
    d = _dims(x, dimensions)
    ordv = {0: 2, 1: 2, 2: 1, 3: float("inf")}.get(int(mode), mode)   # 0 frobenius, 1 euclid, 2 L1, 3 Linf
    return torch.linalg.vector_norm(x, ord=ordv, dim=d)


# ----------------------------------------------------------------------------- cumulative
def _cum(fn):
    def run(x, dimensions=None, exclusive=False, reverse=False, **kw):
        d = _dims(x, dimensions)
        if d is None:
            xx, dd = x.reshape(-1), 0
        else:
            xx, dd = x, d[0]
        if reverse:
            xx = xx.flip(dd)
        r = fn(xx, dd)
        if exclusive:
            ident = 0 if fn is torch.cumsum else 1
            r = torch.cat([torch.full_like(r.narrow(dd, 0, 1), ident), r.narrow(dd, 0, r.shape[dd] - 1)], dd)
        if reverse:
            r = r.flip(dd)
        return r.reshape(x.shape)
    return run


for _n, _f in (("cumsum", torch.cumsum), ("cumprod", torch.cumprod)):
    _run = _cum(_f)
    op(_n)(_run)

    def _mkbp(_run):
        def bp(x, *rest, dimensions=None, exclusive=False, reverse=False, **kw):
            g = rest[-1]
            x = x.detach().requires_grad_(True)
            with torch.enable_grad():
                y = _run(x, dimensions, exclusive, reverse)
            return torch.autograd.grad(y, x, g)[0]
        return bp
    op(_n + "_bp")(_mkbp(_run))


# ----------------------------------------------------------------------------- segment reductions
def _segment(x, ids, num, mode):
    ids = ids.long()
    num = int(num if num is not None else (int(ids.max()) + 1 if ids.numel() else 0))
    shape = (num,) + tuple(x.shape[1:])
    idx = ids.reshape([-1] + [1] * (x.dim() - 1)).expand_as(x)
    if mode in ("sum", "mean", "sqrt_n"):
        out = torch.zeros(shape, dtype=x.dtype, device=x.device).scatter_add_(0, idx, x)
        if mode != "sum":
            cnt = torch.zeros(num, dtype=x.dtype, device=x.device).scatter_add_(0, ids, torch.ones_like(ids, dtype=x.dtype))
            cnt = cnt.clamp_min(1).reshape([-1] + [1] * (x.dim() - 1))
            out = out / (cnt if mode == "mean" else cnt.sqrt())
        return out
    red = {"max": "amax", "min": "amin", "prod": "prod"}[mode]
    init = {"max": -float("inf"), "min": float("inf"), "prod": 1.0}[mode]
    out = torch.full(shape, init, dtype=x.dtype, device=x.device).scatter_reduce(0, idx, x, red, include_self=True)
    if mode in ("max", "min"):
        present = torch.zeros(num, dtype=torch.bool, device=x.device)
        present[ids] = True
        out = torch.where(present.reshape([-1] + [1] * (x.dim() - 1)), out, torch.zeros_like(out))
    return out


for _m in ("sum", "mean", "max", "min", "prod", "sqrt_n"):
    def _mk(_m):
        def seg(x, ids, **kw):
            return _segment(x, ids, None, _m)

        def useg(x, ids, numSegments=None, **kw):
            if isinstance(numSegments, torch.Tensor):
                numSegments = int(numSegments)
            return _segment(x, ids, numSegments, _m)

        def seg_bp(x, ids, g, numSegments=None, **kw):
            xx = x.detach().requires_grad_(True)
            with torch.enable_grad():
                y = _segment(xx, ids, numSegments if not isinstance(numSegments, torch.Tensor) else int(numSegments), _m)
            return torch.autograd.grad(y, xx, g)[0], torch.zeros_like(ids)
        return seg, useg, seg_bp
    _s, _u, _b = _mk(_m)
    if _m != "sqrt_n":
        op(f"segment_{_m}")(_s)
        op(f"segment_{_m}_bp", n_out=2)(_b)
    op(f"unsorted_segment_{_m}")(_u)
    op(f"unsorted_segment_{_m}_bp", n_out=2)(_b)


# ----------------------------------------------------------------------------- selection
@op("top_k", n_out=2, differentiable=False)
def top_k(x, k=1, needSort=True, **kw):
    if isinstance(k, torch.Tensor):
        k = int(k)
    r = torch.topk(x, int(k), dim=-1, sorted=bool(needSort))
    return r.values, r.indices


@op("in_top_k", differentiable=False)
def in_top_k(predictions, targets, k=1, **kw):
    topk = torch.topk(predictions, int(k), dim=-1).indices
    return (topk == targets.long().reshape(-1, 1)).any(dim=1)


@op("nth_element", differentiable=False)
def nth_element(x, n, reverse=False, **kw):
    n = int(n)
    s = torch.sort(x, dim=-1, descending=bool(reverse)).values
    return s[..., n]


@op("percentile", differentiable=False)
def percentile(x, q=50.0, interpolation=2, dimensions=None, keepDims=False, **kw):
    mode = {0: "lower", 1: "higher", 2: "nearest"}.get(int(interpolation), "linear")
    d = _dims(x, dimensions)
    if d is None:
        return torch.quantile(x.reshape(-1).float(), q / 100.0, interpolation=mode).to(x.dtype)
    other = [i for i in range(x.dim()) if i not in d]
    xp = x.permute(*other, *d).reshape([x.shape[i] for i in other] + [-1])
    return torch.quantile(xp.float(), q / 100.0, dim=-1, interpolation=mode, keepdim=False).to(x.dtype)


@op("unique", n_out=2, differentiable=False)
def unique(x, **kw):
    vals, inv = torch.unique(x.reshape(-1), sorted=False, return_inverse=True)
    # first-occurrence order, as the native op
    first = torch.full((vals.numel(),), x.numel(), dtype=torch.long, device=x.device)
    first.scatter_reduce_(0, inv, torch.arange(x.numel(), device=x.device), "amin")
    order = torch.argsort(first)
    remap = torch.empty_like(order)
    remap[order] = torch.arange(order.numel(), device=x.device)
    return vals[order], remap[inv]


@op("unique_with_counts", n_out=3, differentiable=False)
def unique_with_counts(x, **kw):
    v, idx = unique(x)
    cnt = torch.bincount(idx, minlength=v.numel())
    return v, idx, cnt


@op("listdiff", n_out=2, differentiable=False)
def listdiff(x, y, **kw):
    keep = ~torch.isin(x, y)
    return x[keep], torch.nonzero(keep).reshape(-1)


@op("bincount", differentiable=False)
def bincount(x, weights=None, minLength=0, maxLength=None, **kw):
    r = torch.bincount(x.reshape(-1).long(), weights=None if weights is None else weights.reshape(-1), minlength=int(minLength))
    return r[:int(maxLength)] if maxLength else r


@op("histogram", differentiable=False)
def histogram(x, numBins=10, **kw):
    return torch.histc(x.float(), bins=int(numBins)).long()


@op("histogram_fixed_width", differentiable=False)
def histogram_fixed_width(x, range_, nbins=100, **kw):
    lo, hi = float(range_.reshape(-1)[0]), float(range_.reshape(-1)[1])
    nb = int(nbins)
    idx = ((x.float() - lo) / (hi - lo) * nb).floor().clamp(0, nb - 1).long()
    return torch.bincount(idx.reshape(-1), minlength=nb)


@op("zero_fraction", differentiable=False)
def zero_fraction(x, **kw):
    return (x == 0).float().mean()


@op("confusion_matrix", differentiable=False)
def confusion_matrix(labels, pred, weights=None, numClasses=None, **kw):
    n = int(numClasses) if numClasses else int(max(labels.max(), pred.max())) + 1
    idx = labels.long() * n + pred.long()
    w = weights if weights is not None else torch.ones_like(idx)
    return torch.zeros(n * n, dtype=w.dtype, device=labels.device).scatter_add_(0, idx.reshape(-1), w.reshape(-1)).reshape(n, n)


@op("hashcode", differentiable=False)
def hashcode(x, **kw):
    v = x.reshape(-1).contiguous().view(torch.uint8).long()
    h = torch.tensor(0, dtype=torch.int64)
    mult = torch.tensor(31, dtype=torch.int64)
    # polynomial hash evaluated with a running power on the host (small inputs) or in blocks on device
    acc = 0
    for b in v.cpu().tolist():
        acc = (acc * 31 + b) & 0x7FFFFFFFFFFFFFFF
    return torch.tensor(acc, dtype=torch.int64, device=x.device)
