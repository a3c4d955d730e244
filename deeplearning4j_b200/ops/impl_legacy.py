"""Legacy-loop functors that have no declarable-op twin of the same name: the remainder of
``libnd4j/include/loops/legacy_ops.h:27-131`` (functor bodies in ``libnd4j/include/ops/ops.h``), registered so that every
``(op type, opNum)`` pair of a FlatGraph written by the reference resolves to an executable op."""
from __future__ import annotations

import math

import torch

from .registry import op

_EPS = 1e-5


def _t(x, like=None):
    if isinstance(x, torch.Tensor):
        return x
    return torch.as_tensor(x, dtype=like.dtype if like is not None and like.is_floating_point() else None,
                           device=like.device if like is not None else None)


@op("epsilon", group="legacy", differentiable=False)
def epsilon(x, y, eps=_EPS, **kw):
    """``simdOps::Epsilon``: |x - y| <= eps."""
    return (x - _t(y, x)).abs() <= eps


_CONDITIONS = {0: lambda x, c, e: (x - c).abs() <= e, 1: lambda x, c, e: (x - c).abs() > e, 2: lambda x, c, e: x < c,
               3: lambda x, c, e: x > c, 4: lambda x, c, e: x <= c, 5: lambda x, c, e: x >= c, 6: lambda x, c, e: x.abs() < c,
               7: lambda x, c, e: x.abs() > c, 8: lambda x, c, e: torch.isinf(x), 9: lambda x, c, e: torch.isnan(x),
               10: lambda x, c, e: x == c, 11: lambda x, c, e: x != c, 12: lambda x, c, e: x.abs() >= c, 13: lambda x, c, e: x.abs() <= c,
               14: lambda x, c, e: torch.isfinite(x), 15: lambda x, c, e: ~torch.isfinite(x)}


def _cond(x, compare=0.0, eps=_EPS, mode=0):
    return _CONDITIONS[int(mode)](x, compare, eps)


@op("match_condition_transform", "match_condition_bool", group="legacy", differentiable=False)
def match_condition_transform(x, compare=0.0, eps=_EPS, mode=0, **kw):
    """``simdOps::MatchConditionBool``: element-wise condition (``Conditions`` mode ids of ``BooleanIndexing``)."""
    return _cond(x, compare, eps, mode)


@op("amax_pairwise", group="legacy")
def amax_pairwise(x, y, **kw):
    y = _t(y, x)
    return torch.where(x.abs() >= y.abs(), x, y)


@op("amin_pairwise", group="legacy")
def amin_pairwise(x, y, **kw):
    y = _t(y, x)
    return torch.where(x.abs() <= y.abs(), x, y)


@op("is_inf_or_nan", group="legacy", differentiable=False)
def is_inf_or_nan(x, dimensions=None, keepDims=False, **kw):
    r = ~torch.isfinite(x)
    return r if dimensions is None else r.any(dim=tuple(dimensions), keepdim=keepDims)


@op("is_positive", group="legacy", differentiable=False)
def is_positive(x, dimensions=None, keepDims=False, **kw):
    r = x > 0
    return r if dimensions is None else r.all(dim=tuple(dimensions), keepdim=keepDims)


@op("is_negative", group="legacy", differentiable=False)
def is_negative(x, dimensions=None, keepDims=False, **kw):
    r = x < 0
    return r if dimensions is None else r.all(dim=tuple(dimensions), keepdim=keepDims)


@op("scaled_tanh", group="legacy")
def scaled_tanh(x, a=1.7159, b=2.0 / 3.0, **kw):
    return a * torch.tanh(b * x)


@op("tan_derivative", group="legacy")
def tan_derivative(x, **kw):
    return 1.0 / torch.cos(x) ** 2


@op("acosh_derivative", group="legacy")
def acosh_derivative(x, **kw):
    return 1.0 / (torch.sqrt(x - 1.0) * torch.sqrt(x + 1.0))


@op("asinh_derivative", group="legacy")
def asinh_derivative(x, **kw):
    return 1.0 / torch.sqrt(x * x + 1.0)


@op("sinh_derivative", group="legacy")
def sinh_derivative(x, **kw):
    return torch.cosh(x)


@op("log_sigmoid_derivative", group="legacy")
def log_sigmoid_derivative(x, **kw):
    return 1.0 / (torch.exp(x) + 1.0)


@op("special_derivative", group="legacy")
def special_derivative(x, **kw):
    """``simdOps::SpecialDerivative``: x (1 - x)."""
    return x * (1.0 - x)


@op("stabilize_fp16", group="legacy")
def stabilize_fp16(x, **kw):
    """``simdOps::StabilizeFP16``: floors magnitudes below the fp16 denormal range."""
    return torch.where(x.abs() < 6e-5, torch.full_like(x, 6e-5) * torch.sign(x + (x == 0)), x)


@op("remainder", group="legacy")
def remainder(x, y, **kw):
    return torch.remainder(x, _t(y, x))


@op("fmod", group="legacy")
def fmod(x, y, **kw):
    return torch.fmod(x, _t(y, x))


@op("truncatemod", "truncate_mod", group="legacy")
def truncatemod(x, y, **kw):
    return torch.fmod(x, _t(y, x))


@op("compare_and_set", group="legacy")
def compare_and_set(x, y=None, compare=0.0, set=0.0, eps=_EPS, mode=0, **kw):
    """``simdOps::CompareAndSet``: where the condition holds for x take ``set`` (scalar form) or y (pairwise form)."""
    m = _cond(x, compare, eps, mode)
    return torch.where(m, _t(set, x).to(x.dtype) if y is None else _t(y, x), x)


@op("compare_and_replace", group="legacy")
def compare_and_replace(x, y, compare=0.0, eps=_EPS, mode=0, **kw):
    """``simdOps::CompareAndReplace``: where the condition holds for x take y."""
    return torch.where(_cond(x, compare, eps, mode), _t(y, x), x)


@op("sxe_logits_smoother", group="legacy")
def sxe_logits_smoother(x, smoothing=0.0, numClasses=None, **kw):
    """``simdOps::SXELogitsSmoother``: label smoothing x (1 - s) + s / classes (classes = last axis by default)."""
    n = numClasses if numClasses is not None else x.shape[-1]
    return x * (1.0 - smoothing) + smoothing / n


@op("log_x", group="legacy")
def log_x(x, base=math.e, **kw):
    return torch.log(x) / math.log(base)


@op("lstm_clip", group="legacy")
def lstm_clip(x, clip=0.0, **kw):
    return x if not clip else x.clamp(-clip, clip)


@op("squared_reverse_subtract", group="legacy")
def squared_reverse_subtract(x, y, **kw):
    return (_t(y, x) - x) ** 2


@op("reverse_pow", group="legacy")
def reverse_pow(x, y, **kw):
    return torch.pow(_t(y, x), x)


@op("reduce_normp", group="legacy")
def reduce_normp(x, dimensions=None, keepDims=False, p=2.0, **kw):
    d = None if dimensions is None else tuple(dimensions)
    return x.abs().pow(p).sum(dim=d, keepdim=keepDims).pow(1.0 / p) if d is not None else x.abs().pow(p).sum().pow(1.0 / p)


@op("probablistic_merge", group="legacy", differentiable=False)
def probablistic_merge(x, y, prob=0.5, seed=None, **kw):
    """``randomOps::ProbablisticMerge``: each element from x with probability ``prob``, else from y."""
    g = None if seed is None else torch.Generator(device=x.device).manual_seed(int(seed))
    return torch.where(torch.rand(x.shape, device=x.device, generator=g) < prob, x, y)


@op("random_binomial", "binomial_distribution_ex", group="legacy", differentiable=False)
def random_binomial(*a, shape=None, trials=1, prob=0.5, seed=None, dtype=torch.float32, device=None, **kw):
    shape = tuple(int(s) for s in (shape if shape is not None else a[0].tolist()))
    g = None if seed is None else torch.Generator().manual_seed(int(seed))
    r = (torch.rand((int(trials),) + shape, generator=g) < prob).sum(0)
    return r.to(dtype).to(device) if device is not None else r.to(dtype)


@op("random_lognormal", group="legacy", differentiable=False)
def random_lognormal(*a, shape=None, mean=0.0, stddev=1.0, seed=None, dtype=torch.float32, device=None, **kw):
    shape = tuple(int(s) for s in (shape if shape is not None else a[0].tolist()))
    g = None if seed is None else torch.Generator().manual_seed(int(seed))
    r = torch.exp(torch.randn(shape, generator=g) * stddev + mean).to(dtype)
    return r.to(device) if device is not None else r


@op("random_truncated_normal", group="legacy", differentiable=False)
def random_truncated_normal(*a, shape=None, mean=0.0, stddev=1.0, seed=None, dtype=torch.float32, device=None, **kw):
    shape = tuple(int(s) for s in (shape if shape is not None else a[0].tolist()))
    g = None if seed is None else torch.Generator().manual_seed(int(seed))
    r = torch.empty(shape)
    torch.nn.init.trunc_normal_(r, mean, stddev, mean - 2 * stddev, mean + 2 * stddev, generator=g)
    return r.to(dtype).to(device) if device is not None else r.to(dtype)


@op("exponential_distribution_inv", group="legacy", differentiable=False)
def exponential_distribution_inv(x, lam=1.0, **kw):
    """``randomOps::ExponentialDistributionInv``: inverse CDF applied to uniform samples x."""
    return -torch.log(1.0 - x) / lam


@op("relative_error", group="legacy")
def relative_error(x, y, **kw):
    y = _t(y, x)
    d = x.abs() + y.abs()
    return torch.where(d == 0, torch.zeros_like(x), (x - y).abs() / d)


@op("binary_relative_error", group="legacy", differentiable=False)
def binary_relative_error(x, y, threshold=0.0, **kw):
    return (relative_error(x, y) > threshold).to(x.dtype)


@op("binary_min_abs_relative_error", group="legacy", differentiable=False)
def binary_min_abs_relative_error(x, y, thresholdRelative=0.0, thresholdAbsolute=0.0, **kw):
    y = _t(y, x)
    bad = (relative_error(x, y) > thresholdRelative) & ((x - y).abs() > thresholdAbsolute)
    return bad.to(x.dtype)


@op("log_poisson_loss_full", group="legacy")
def log_poisson_loss_full(x, y, **kw):
    """``simdOps::LogPoissonLossFull``: exp(y) - x y + x log x - x + 0.5 log(2 pi x) (labels x, log-predictions y)."""
    y = _t(y, x)
    st = x * torch.log(x.clamp_min(1e-30)) - x + 0.5 * torch.log((2 * math.pi * x).clamp_min(1e-30))
    return torch.exp(y) - x * y + torch.where(x > 1.0, st, torch.zeros_like(st))


@op("match_condition", group="legacy", differentiable=False)
def match_condition(x, y=None, dimensions=None, keepDims=False, compare=0.0, eps=_EPS, mode=0, **kw):
    """``simdOps::MatchCondition``: as a reduction (REDUCE_LONG) the number of elements that satisfy the condition, as a
    pairwise / scalar boolean op (a second operand given) the element-wise condition against that operand."""
    if y is not None:
        return _cond(x, _t(y, x), eps, mode)
    m = _cond(x, compare, eps, mode).to(torch.int64)
    if dimensions is None:
        return m.sum()
    return m.sum(dim=tuple(dimensions), keepdim=keepDims)
