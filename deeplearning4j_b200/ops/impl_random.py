"""Random ops (``headers/random.h`` + legacy RANDOM_OPS, ``loops/legacy_ops.h:108-113``).

The reference's counter-based xoroshiro generator (``graph/RandomGenerator.h``) is replaced by
torch's Philox streams: draws are reproducible per (seed, device) but not bit-identical to the JVM."""
from __future__ import annotations

import torch

from ..nd.dtype import DataType
from .registry import op

_STATE = {"seed": 119, "gens": {}}


def _gen(device):
    key = str(device)
    g = _STATE["gens"].get(key)
    if g is None:
        g = torch.Generator(device=device)
        g.manual_seed(_STATE["seed"])
        _STATE["gens"][key] = g
    return g


def _shape(s):
    if isinstance(s, torch.Tensor):
        return [int(v) for v in s.reshape(-1).tolist()]
    return [int(v) for v in s]


def _td(dtype, default=torch.float32):
    if dtype is None:
        return default
    if isinstance(dtype, torch.dtype):
        return dtype
    return DataType(dtype).to_torch() if not isinstance(dtype, str) else DataType.from_name(dtype).to_torch()


@op("set_seed", differentiable=False)
def set_seed(seed=119, **kw):
    s = int(seed.reshape(-1)[0]) if isinstance(seed, torch.Tensor) else int(seed)
    _STATE["seed"] = s
    _STATE["gens"].clear()
    return torch.tensor(s, dtype=torch.int64)


op("get_seed", differentiable=False)(lambda **kw: torch.tensor(_STATE["seed"], dtype=torch.int64))


@op("randomuniform", "random_uniform", "distribution_uniform", differentiable=False)
def randomuniform(shape, min=0.0, max=1.0, dtype=None, device="cpu", **kw):
    dt = _td(dtype)
    if not dt.is_floating_point:
        return torch.randint(int(min), int(max), _shape(shape), generator=_gen(device), device=device, dtype=dt)
    return torch.rand(_shape(shape), generator=_gen(device), device=device, dtype=dt) * (max - min) + min


@op("random_normal", "distribution_gaussian", differentiable=False)
def random_normal(shape, mean=0.0, stdev=1.0, dtype=None, device="cpu", **kw):
    return torch.randn(_shape(shape), generator=_gen(device), device=device, dtype=_td(dtype)) * stdev + mean


@op("random_bernoulli", "distribution_bernoulli", differentiable=False)
def random_bernoulli(shape, p=0.5, dtype=None, device="cpu", **kw):
    return (torch.rand(_shape(shape), generator=_gen(device), device=device) < p).to(_td(dtype))


@op("random_exponential", "distribution_exponential", differentiable=False)
def random_exponential(shape, lambda_=1.0, dtype=None, device="cpu", **kw):
    lam = kw.get("lambda", lambda_)
    u = torch.rand(_shape(shape), generator=_gen(device), device=device, dtype=_td(dtype))
    return -torch.log1p(-u) / lam


@op("distribution_lognormal", differentiable=False)
def distribution_lognormal(shape, mean=0.0, stdev=1.0, dtype=None, device="cpu", **kw):
    return torch.exp(random_normal(shape, mean, stdev, dtype, device))


@op("distribution_truncated", "distribution_truncatednormal", differentiable=False)
def distribution_truncated(shape, mean=0.0, stdev=1.0, dtype=None, device="cpu", **kw):
    out = torch.empty(_shape(shape), device=device, dtype=_td(dtype))
    torch.nn.init.trunc_normal_(out, mean, stdev, mean - 2 * stdev, mean + 2 * stdev, generator=_gen(device))
    return out


@op("distribution_binomial", "distribution_binomial_ex", differentiable=False)
def distribution_binomial(shape, trials=1, p=0.5, dtype=None, device="cpu", **kw):
    s = _shape(shape)
    acc = torch.zeros(s, device=device, dtype=_td(dtype))
    for _ in range(int(trials)):
        acc += (torch.rand(s, generator=_gen(device), device=device) < p).to(acc.dtype)
    return acc


@op("random_gamma", differentiable=False)
def random_gamma(shape, alpha, beta=None, **kw):
    a = alpha.float()
    b = beta.float() if beta is not None else torch.ones_like(a)
    s = _shape(shape) + list(torch.broadcast_shapes(a.shape, b.shape))
    return torch.distributions.Gamma(a.expand(s), b.expand(s)).sample()


@op("random_poisson", differentiable=False)
def random_poisson(shape, lam, **kw):
    s = _shape(shape) + list(lam.shape)
    return torch.poisson(lam.float().expand(s), generator=_gen(lam.device))


@op("random_multinomial", differentiable=False)
def random_multinomial(logits, numSamples, dimC=-1, dtype=None, **kw):
    n = int(numSamples.reshape(-1)[0]) if isinstance(numSamples, torch.Tensor) else int(numSamples)
    lg = logits if int(dimC) in (-1, logits.dim() - 1) else logits.transpose(int(dimC), -1)
    return torch.multinomial(torch.softmax(lg.float(), -1), n, replacement=True, generator=_gen(logits.device)).to(_td(dtype, torch.int64))


@op("random_shuffle", differentiable=False)
def random_shuffle(x, **kw):
    return x[torch.randperm(x.shape[0], generator=_gen("cpu")).to(x.device)]


@op("random_crop", differentiable=False)
def random_crop(x, shape, seed=None, **kw):
    s = _shape(shape)
    idx = tuple(slice(o, o + n) for o, n in ((int(torch.randint(0, x.shape[i] - s[i] + 1, (), generator=_gen("cpu"))), s[i]) for i in range(len(s))))
    return x[idx]


@op("dropout_random", "random_dropout")
def dropout_random(x, p=0.5, **kw):
    keep = (torch.rand(x.shape, generator=_gen(x.device), device=x.device) < p).to(x.dtype)
    return x * keep


@op("alpha_dropout")
def alpha_dropout(x, p=0.5, a=1.0, alphaPrime=-1.7580993408473766, b=0.0, **kw):
    keep = torch.rand(x.shape, generator=_gen(x.device), device=x.device) < p
    return a * torch.where(keep, x, torch.full_like(x, alphaPrime)) + b


@op("choice", differentiable=False)
def choice(source, probs, numSamples=1, **kw):
    idx = torch.multinomial(probs.float().reshape(-1), int(numSamples), replacement=True, generator=_gen(probs.device))
    return source.reshape(-1)[idx]
