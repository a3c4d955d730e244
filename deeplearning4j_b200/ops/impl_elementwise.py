"""Elementwise ops: activations (``headers/activations.h``), broadcastable arithmetic / comparison
(``headers/broadcastable.h``), boolean (``headers/boolean.h``), bitwise (``headers/bitwise.h``),
datatype casts (``headers/datatypes.h``) and the legacy transform / pairwise / scalar families
(``libnd4j/include/loops/legacy_ops.h:27-131``).  ``*_bp`` ops return input gradients given the
upstream gradient as the last input, matching the native signatures."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ..nd.dtype import DataType
from .registry import op


def _bp(fn):
    """Generic backprop through ``fn`` for a single differentiable input."""
    def run(x, grad, **kw):
        x = x.detach().requires_grad_(True)
        with torch.enable_grad():
            y = fn(x, **kw)
        return torch.autograd.grad(y, x, grad)[0]
    return run


def _unary(name, fn, *aliases, bp=True):
    op(name, *aliases)(lambda x, **kw: fn(x))
    if bp:
        op(name + "_bp")(_bp(lambda x, **kw: fn(x)))


# ----------------------------------------------------------------------------- activations
def _rational_tanh(x):
    y = x * (2.0 / 3.0)
    a = y.abs()
    return 1.7159 * torch.sign(y) * (1.0 - 1.0 / (1.0 + a + y * y + 1.41645 * y ** 4))


_unary("sigmoid", torch.sigmoid)
_unary("softsign", F.softsign)
_unary("tanh", torch.tanh)
_unary("softplus", F.softplus)
_unary("relu6", F.relu6)
_unary("selu", F.selu)
_unary("cube", lambda x: x * x * x)
_unary("rectifiedtanh", lambda x: F.relu(torch.tanh(x)))
_unary("rationaltanh", _rational_tanh)
_unary("hardtanh", F.hardtanh)
_unary("hardsigmoid", lambda x: torch.clamp(0.2 * x + 0.5, 0, 1))
_unary("identity", lambda x: x)
# libnd4j ops.h: GELU = x * sigmoid(1.702 x); PreciseGELU = 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
_unary("gelu", lambda x: x * torch.sigmoid(1.702 * x))
_unary("precise_gelu", lambda x: F.gelu(x, approximate="tanh"))
_unary("gelu_erf", F.gelu)
_unary("swish", F.silu)
_unary("mish", F.mish)


@op("relu")
def relu(x, cutoff=0.0, **kw):
    return torch.where(x > cutoff, x, torch.zeros_like(x)) if cutoff else F.relu(x)


op("relu_bp")(lambda x, g, cutoff=0.0, **kw: g * (x > cutoff).to(g.dtype))
op("lrelu", "leakyrelu")(lambda x, alpha=0.01, **kw: F.leaky_relu(x, alpha))
op("lrelu_bp")(lambda x, g, alpha=0.01, **kw: g * torch.where(x > 0, torch.ones_like(x), torch.full_like(x, alpha)))
op("elu")(lambda x, alpha=1.0, **kw: F.elu(x, alpha))
op("elu_bp")(_bp(lambda x, alpha=1.0, **kw: F.elu(x, alpha)))
op("thresholdedrelu")(lambda x, theta=1.0, **kw: torch.where(x > theta, x, torch.zeros_like(x)))
op("thresholdedrelu_bp")(lambda x, g, theta=1.0, **kw: g * (x > theta).to(g.dtype))
op("crelu")(lambda x, **kw: torch.cat([F.relu(x), F.relu(-x)], dim=-1))
op("crelu_bp")(_bp(lambda x, **kw: torch.cat([F.relu(x), F.relu(-x)], dim=-1)))
op("identity_n", n_out=-1)(lambda *xs, **kw: tuple(xs))


@op("prelu")
def prelu(x, alpha, sharedAxes=None, **kw):
    a = alpha
    while a.dim() < x.dim():
        a = a.unsqueeze(0)
    return torch.where(x >= 0, x, x * a)


@op("prelu_bp", n_out=2)
def prelu_bp(x, alpha, g, **kw):
    x = x.detach().requires_grad_(True)
    alpha = alpha.detach().requires_grad_(True)
    with torch.enable_grad():
        y = prelu(x, alpha)
    return torch.autograd.grad(y, (x, alpha), g)


# ----------------------------------------------------------------------------- broadcastable
def _binary(name, fn, *aliases, bp=True):
    op(name, *aliases)(lambda x, y, **kw: fn(x, y))
    if bp:
        @op(name + "_bp", n_out=2)
        def _b(x, y, g, **kw):
            x = x.detach().requires_grad_(True)
            y = y.detach().requires_grad_(True)
            with torch.enable_grad():
                z = fn(x, y)
            gx, gy = torch.autograd.grad(z, (x, y), g, allow_unused=True)
            return (gx if gx is not None else torch.zeros_like(x)), (gy if gy is not None else torch.zeros_like(y))


def _t(v, like):
    return v if isinstance(v, torch.Tensor) else torch.as_tensor(v, dtype=like.dtype, device=like.device)


_binary("add", lambda x, y: x + y)
_binary("subtract", lambda x, y: x - y, "sub")
_binary("multiply", lambda x, y: x * y, "mul")
_binary("divide", lambda x, y: x / y, "div")
_binary("reversesubtract", lambda x, y: y - x, "rsub")
_binary("reversedivide", lambda x, y: y / x, "rdiv")
_binary("squaredsubtract", lambda x, y: (x - y) ** 2)
_binary("maximum", torch.maximum, "max_pairwise")
_binary("minimum", torch.minimum, "min_pairwise")
_binary("floormod", lambda x, y: torch.remainder(x, y))
_binary("mod", lambda x, y: torch.remainder(x, y))      # simdOps::Mod is d1 - floor(d1 / d2) * d2 (ops.h:1708), not C fmod
_binary("reversemod", lambda x, y: torch.fmod(y, x))
_binary("floordiv", lambda x, y: torch.floor_divide(x, y))
# piecewise constant: both gradients are zero (floordiv.cpp: floordiv_bp assigns 0 to gradX and gradY)
op("floordiv_bp", n_out=2)(lambda x, y, g, **kw: (torch.zeros_like(x), torch.zeros_like(_t(y, x)).expand_as(torch.broadcast_tensors(x, _t(y, x))[1]).clone()
                                                  if not isinstance(y, torch.Tensor) else torch.zeros_like(y)))
_binary("realdiv", lambda x, y: x / y)
_binary("Pow", lambda x, y: torch.pow(x, y), "pow_pairwise")
_binary("assign", lambda x, y: y.expand_as(x).clone() if y.shape != x.shape else y.clone())
op("truncatediv")(lambda x, y, **kw: torch.trunc(x / y).to(x.dtype))
op("divide_no_nan")(lambda x, y, **kw: torch.where(y == 0, torch.zeros_like(x), x / torch.where(y == 0, torch.ones_like(y), y)))
op("tf_atan2", "atan2")(lambda y, x, **kw: torch.atan2(y, x))
op("igamma")(lambda a, x, **kw: torch.special.gammainc(a, x))
op("igammac")(lambda a, x, **kw: torch.special.gammaincc(a, x))
op("axpy")(lambda x, y, a=1.0, **kw: a * x + y)

for _n, _f in (("equals", torch.eq), ("not_equals", torch.ne), ("less", torch.lt), ("less_equal", torch.le),
               ("greater", torch.gt), ("greater_equal", torch.ge)):
    op(_n, differentiable=False)(lambda x, y, _f=_f, **kw: _f(x, _t(y, x)))
op("boolean_and", differentiable=False)(lambda x, y, **kw: torch.logical_and(x != 0, y != 0))
op("boolean_or", differentiable=False)(lambda x, y, **kw: torch.logical_or(x != 0, y != 0))
op("boolean_xor", differentiable=False)(lambda x, y, **kw: torch.logical_xor(x != 0, y != 0))
op("boolean_not", "not", differentiable=False)(lambda x, **kw: x == 0)

for _n, _f in (("lt_scalar", torch.lt), ("gt_scalar", torch.gt), ("lte_scalar", torch.le), ("gte_scalar", torch.ge),
               ("eq_scalar", torch.eq), ("neq_scalar", torch.ne)):
    op(_n, differentiable=False)(lambda x, y, _f=_f, **kw: _f(x, _t(y, x)).all())

op("Where", "where", differentiable=False, n_out=-1)(
    lambda c, *xy, **kw: torch.where(c.bool(), xy[0], xy[1]) if xy else tuple(torch.nonzero(c, as_tuple=False).unbind(1)))
op("where_np")(lambda c, x=None, y=None, **kw: torch.where(c.bool(), x, y) if x is not None else torch.nonzero(c))
op("select")(lambda c, x, y, **kw: torch.where(c.bool(), x, y))
op("is_non_decreasing", differentiable=False)(lambda x, **kw: (x.reshape(-1)[1:] >= x.reshape(-1)[:-1]).all())
op("is_strictly_increasing", differentiable=False)(lambda x, **kw: (x.reshape(-1)[1:] > x.reshape(-1)[:-1]).all())
op("is_numeric_tensor", differentiable=False)(lambda x, **kw: torch.tensor(x.dtype != torch.bool))


@op("choose", n_out=2, differentiable=False)
def choose(x, comp=None, mode=0, scalar=0.0, **kw):
    c = comp if comp is not None else torch.as_tensor(scalar, dtype=x.dtype, device=x.device)
    fns = [torch.eq, torch.ne, torch.lt, torch.gt, torch.le, torch.ge]
    m = fns[int(mode) % 6](x, c)
    return x[m], m.sum()


# ----------------------------------------------------------------------------- bitwise
op("bitwise_and", differentiable=False)(lambda x, y, **kw: torch.bitwise_and(x, y))
op("bitwise_or", differentiable=False)(lambda x, y, **kw: torch.bitwise_or(x, y))
op("bitwise_xor", differentiable=False)(lambda x, y, **kw: torch.bitwise_xor(x, y))
op("toggle_bits", differentiable=False)(lambda x, **kw: torch.bitwise_not(x))
op("shift_bits", differentiable=False)(lambda x, s, **kw: torch.bitwise_left_shift(x, _t(s, x)))
op("rshift_bits", differentiable=False)(lambda x, s, **kw: torch.bitwise_right_shift(x, _t(s, x)))


def _bits_of(x):
    return x.element_size() * 8


@op("cyclic_shift_bits", differentiable=False)
def cyclic_shift_bits(x, s, **kw):
    n = _bits_of(x)
    s = _t(s, x) % n
    ux = x.to(torch.int64) & ((1 << n) - 1) if n < 64 else x
    r = ((ux << s) | (ux >> (n - s))) & ((1 << n) - 1) if n < 64 else (x << s) | ((x >> (n - s)) & ((1 << s) - 1))
    return r.to(x.dtype)


@op("cyclic_rshift_bits", differentiable=False)
def cyclic_rshift_bits(x, s, **kw):
    n = _bits_of(x)
    return cyclic_shift_bits(x, (n - _t(s, x)) % n)


@op("bits_hamming_distance", differentiable=False)
def bits_hamming_distance(x, y, **kw):
    v = torch.bitwise_xor(x, y).to(torch.int64)
    cnt = torch.zeros_like(v)
    for i in range(_bits_of(x)):
        cnt += (v >> i) & 1
    return cnt.sum()


# ----------------------------------------------------------------------------- casts
for _n, _dt in (("to_double", torch.float64), ("to_float16", torch.float16), ("to_float32", torch.float32),
                ("to_int32", torch.int32), ("to_int64", torch.int64), ("to_uint32", torch.uint32), ("to_uint64", torch.uint64)):
    op(_n)(lambda x, _dt=_dt, **kw: x.to(_dt))


@op("cast")
def cast(x, dtype=None, dst=None, **kw):
    d = dtype if dtype is not None else dst
    if isinstance(d, int):
        d = DataType(d)
    if isinstance(d, str):
        d = DataType.from_name(d)
    return x.to(d.to_torch() if isinstance(d, DataType) else d)


@op("bitcast", differentiable=False)
def bitcast(x, dtype=None, **kw):
    d = DataType(dtype) if isinstance(dtype, int) else dtype
    return x.contiguous().view(d.to_torch() if isinstance(d, DataType) else d)


op("min_max_datatype", differentiable=False)(
    lambda dtype=DataType.FLOAT, minOrMax=0, **kw: torch.tensor(
        (torch.finfo if DataType(dtype).is_fp() else torch.iinfo)(DataType(dtype).to_torch()).max if minOrMax
        else (torch.finfo if DataType(dtype).is_fp() else torch.iinfo)(DataType(dtype).to_torch()).min))

# ----------------------------------------------------------------------------- legacy transforms (same / strict / float / any / bool)
_TRANSFORMS = {
    "abs": torch.abs, "neg": torch.neg, "sign": torch.sign, "ceil": torch.ceil, "floor": torch.floor, "Floor": torch.floor,
    "round": torch.round, "rint": torch.round, "square": torch.square, "sqrt": torch.sqrt, "rsqrt": torch.rsqrt,
    "exp": torch.exp, "expm1": torch.expm1, "log": torch.log, "log1p": torch.log1p, "Log1p": torch.log1p,
    "log2": torch.log2, "log10": torch.log10, "sin": torch.sin, "cos": torch.cos, "tan": torch.tan,
    "asin": torch.asin, "acos": torch.acos, "atan": torch.atan, "sinh": torch.sinh, "cosh": torch.cosh,
    "asinh": torch.asinh, "acosh": torch.acosh, "atanh": torch.atanh, "erf": torch.erf, "erfc": torch.erfc,
    "reciprocal": torch.reciprocal, "oneminus": lambda x: 1 - x, "onesas": torch.ones_like,
    "timesoneminus": lambda x: x * (1 - x), "sigmoid_derivative": lambda x: torch.sigmoid(x) * (1 - torch.sigmoid(x)),
    "tanh_derivative": lambda x: 1 - torch.tanh(x) ** 2, "softsign_derivative": lambda x: 1 / (1 + x.abs()) ** 2,
    "hardtanh_derivative": lambda x: ((x >= -1) & (x <= 1)).to(x.dtype), "cube_derivative": lambda x: 3 * x * x,
    "lgamma": torch.lgamma, "digamma": torch.digamma, "trunc": torch.trunc, "stabilize": lambda x: x.clamp(-50, 50),
    "affine": lambda x: x, "isnan": torch.isnan, "isinf": torch.isinf, "isfinite": torch.isfinite,
    "ones_as": torch.ones_like, "zeros_as": torch.zeros_like, "zeroslike": torch.zeros_like, "oneslike": torch.ones_like,
    "logsigmoid": F.logsigmoid, "hard_swish": F.hardswish, "softmax_derivative": lambda x: torch.softmax(x, -1) * (1 - torch.softmax(x, -1)),
}
for _n, _f in _TRANSFORMS.items():
    op(_n, differentiable=_n not in ("isnan", "isinf", "isfinite"))(lambda x, _f=_f, **kw: _f(x))

op("pow")(lambda x, p=2.0, **kw: torch.pow(x, p))
op("pow_derivative")(lambda x, p=2.0, **kw: p * torch.pow(x, p - 1))
op("step")(lambda x, cutoff=0.0, **kw: (x > cutoff).to(x.dtype))
op("clipbyvalue", "clip_by_value")(lambda x, clipValueMin=None, clipValueMax=None, **kw: torch.clamp(x, clipValueMin, clipValueMax))
op("replace_nans")(lambda x, value=0.0, **kw: torch.nan_to_num(x, nan=value))
op("set_range")(lambda x, min=0.0, max=1.0, **kw: torch.clamp(x, min, max))
op("zeta")(lambda x, q, **kw: torch.special.zeta(x, q))
op("polygamma")(lambda n, x, **kw: torch.special.polygamma(int(n.reshape(-1)[0]) if isinstance(n, torch.Tensor) else int(n), x))
op("betainc")(lambda a, b, x, **kw: _betainc(a, b, x))
op("check_numerics", differentiable=False)(lambda x, message="", **kw: _check_numerics(x, message))


def _check_numerics(x, message):
    if not torch.isfinite(x).all():
        raise FloatingPointError(f"check_numerics failed: {message}")
    return x


def _betainc(a, b, x, n=200):
    """Regularised incomplete beta via the continued fraction (Lentz), vectorised."""
    a, b, x = torch.broadcast_tensors(a.double(), b.double(), x.double())
    swap = x > (a + 1) / (a + b + 2)
    aa, bb, xx = torch.where(swap, b, a), torch.where(swap, a, b), torch.where(swap, 1 - x, x)
    tiny = 1e-300
    qab, qap, qam = aa + bb, aa + 1, aa - 1
    c = torch.ones_like(xx)
    d = 1 - qab * xx / qap
    d = torch.where(d.abs() < tiny, torch.full_like(d, tiny), d)
    d = 1 / d
    h = d.clone()
    for m in range(1, n):
        m2 = 2 * m
        t = m * (bb - m) * xx / ((qam + m2) * (aa + m2))
        d = 1 + t * d; d = torch.where(d.abs() < tiny, torch.full_like(d, tiny), d)
        c = 1 + t / c; c = torch.where(c.abs() < tiny, torch.full_like(c, tiny), c)
        d = 1 / d; h = h * d * c
        t = -(aa + m) * (qab + m) * xx / ((aa + m2) * (qap + m2))
        d = 1 + t * d; d = torch.where(d.abs() < tiny, torch.full_like(d, tiny), d)
        c = 1 + t / c; c = torch.where(c.abs() < tiny, torch.full_like(c, tiny), c)
        d = 1 / d; h = h * d * c
    lbeta = torch.lgamma(aa) + torch.lgamma(bb) - torch.lgamma(aa + bb)
    front = torch.exp(aa * torch.log(xx.clamp_min(tiny)) + bb * torch.log((1 - xx).clamp_min(tiny)) - lbeta) / aa
    r = front * h
    r = torch.where(swap, 1 - r, r)
    return torch.where(x <= 0, torch.zeros_like(r), torch.where(x >= 1, torch.ones_like(r), r)).to(torch.float32)


# ----------------------------------------------------------------------------- legacy scalar ops
_SCALAR = {"add_scalar": lambda x, s: x + s, "sub_scalar": lambda x, s: x - s, "mul_scalar": lambda x, s: x * s,
           "div_scalar": lambda x, s: x / s, "rsub_scalar": lambda x, s: s - x, "rdiv_scalar": lambda x, s: s / x,
           "max_scalar": lambda x, s: torch.clamp_min(x, s), "min_scalar": lambda x, s: torch.clamp_max(x, s),
           "pow_scalar": lambda x, s: torch.pow(x, s), "fmod_scalar": lambda x, s: torch.fmod(x, s),
           "set_scalar": lambda x, s: torch.full_like(x, s), "mod_scalar": lambda x, s: torch.remainder(x, s)}
for _n, _f in _SCALAR.items():
    op(_n)(lambda x, scalar=0.0, _f=_f, **kw: _f(x, scalar))
