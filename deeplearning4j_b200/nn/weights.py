"""Weight initialisation (``deeplearning4j-nn/.../nn/weights/WeightInit*.java`` and the SameDiff
``org.nd4j.weightinit.impl.*InitScheme`` family) plus the ``Distribution`` configs.

``init(fanIn, fanOut, shape, order, out)`` fills ``out`` (a view of the flat parameter buffer)
in place.  Random draws come from the torch Philox generator of the target device; draw order
(and therefore bit patterns) intentionally differs from the JVM RNG.
"""
from __future__ import annotations

import math

import torch

_PKG = "org.deeplearning4j.nn.weights."
_DPKG = "org.deeplearning4j.nn.conf.distribution."


# --------------------------------------------------------------------------- distributions
class Distribution:
    JAVA = ""; FIELDS: tuple = ()
    def sample_(self, out, gen): raise NotImplementedError
    def to_json(self):
        d = {"@class": _DPKG + self.JAVA}
        for f in self.FIELDS:
            d[f] = getattr(self, f)
        return d
    def __eq__(self, o): return type(self) is type(o) and self.to_json() == o.to_json()
    def __hash__(self): return hash(type(self))


class NormalDistribution(Distribution):
    JAVA = "NormalDistribution"; FIELDS = ("mean", "std")
    def __init__(self, mean=0.0, std=1.0): self.mean, self.std = float(mean), float(std)
    def sample_(self, out, gen): out.normal_(self.mean, self.std, generator=gen)


GaussianDistribution = NormalDistribution


class UniformDistribution(Distribution):
    JAVA = "UniformDistribution"; FIELDS = ("lower", "upper")
    def __init__(self, lower=0.0, upper=1.0): self.lower, self.upper = float(lower), float(upper)
    def sample_(self, out, gen): out.uniform_(self.lower, self.upper, generator=gen)


class TruncatedNormalDistribution(Distribution):
    JAVA = "TruncatedNormalDistribution"; FIELDS = ("mean", "std")
    def __init__(self, mean=0.0, std=1.0): self.mean, self.std = float(mean), float(std)
    def sample_(self, out, gen):
        torch.nn.init.trunc_normal_(out, self.mean, self.std, self.mean - 2 * self.std, self.mean + 2 * self.std, generator=gen)


class LogNormalDistribution(Distribution):
    JAVA = "LogNormalDistribution"; FIELDS = ("mean", "std")
    def __init__(self, mean=0.0, std=1.0): self.mean, self.std = float(mean), float(std)
    def sample_(self, out, gen): out.log_normal_(self.mean, self.std, generator=gen)


class BinomialDistribution(Distribution):
    JAVA = "BinomialDistribution"; FIELDS = ("numberOfTrials", "probabilityOfSuccess")
    def __init__(self, numberOfTrials=1, probabilityOfSuccess=0.5):
        self.numberOfTrials, self.probabilityOfSuccess = int(numberOfTrials), float(probabilityOfSuccess)
    def sample_(self, out, gen):
        acc = torch.zeros_like(out)
        for _ in range(self.numberOfTrials):
            acc += (torch.rand(out.shape, generator=gen, device=out.device) < self.probabilityOfSuccess).to(out.dtype)
        out.copy_(acc)


class ConstantDistribution(Distribution):
    JAVA = "ConstantDistribution"; FIELDS = ("value",)
    def __init__(self, value=0.0): self.value = float(value)
    def sample_(self, out, gen): out.fill_(self.value)


class OrthogonalDistribution(Distribution):
    JAVA = "OrthogonalDistribution"; FIELDS = ("gain",)
    def __init__(self, gain=1.0): self.gain = float(gain)
    def sample_(self, out, gen):
        flat = out.reshape(out.shape[0], -1)
        a = torch.randn(flat.shape, generator=gen, device=out.device, dtype=torch.float32)
        q, r = torch.linalg.qr(a if flat.shape[0] >= flat.shape[1] else a.t())
        q = q * torch.sign(torch.diagonal(r)).unsqueeze(0)
        q = q if flat.shape[0] >= flat.shape[1] else q.t()
        out.copy_((self.gain * q).reshape(out.shape).to(out.dtype))


DISTRIBUTIONS = {c.JAVA: c for c in (NormalDistribution, UniformDistribution, TruncatedNormalDistribution,
                                     LogNormalDistribution, BinomialDistribution, ConstantDistribution,
                                     OrthogonalDistribution)}
DISTRIBUTIONS["GaussianDistribution"] = NormalDistribution


def distribution_from_json(d):
    if d is None:
        return None
    cls = DISTRIBUTIONS[d["@class"].rsplit(".", 1)[-1]]
    return cls(**{k: v for k, v in d.items() if k != "@class"})


# --------------------------------------------------------------------------- weight init
class IWeightInit:
    JAVA = ""
    def init(self, fanIn, fanOut, out: torch.Tensor, gen=None): raise NotImplementedError
    def to_json(self): return {"@class": _PKG + self.JAVA}
    def __eq__(self, o): return type(self) is type(o) and self.to_json() == o.to_json()
    def __hash__(self): return hash(type(self))
    def __repr__(self): return self.JAVA


def _normal(std_fn):
    def init(self, fanIn, fanOut, out, gen=None):
        out.normal_(0.0, std_fn(fanIn, fanOut), generator=gen)
    return init


def _uniform(bound_fn):
    def init(self, fanIn, fanOut, out, gen=None):
        b = bound_fn(fanIn, fanOut)
        out.uniform_(-b, b, generator=gen)
    return init


def _trunc(std_fn):
    def init(self, fanIn, fanOut, out, gen=None):
        s = std_fn(fanIn, fanOut)
        torch.nn.init.trunc_normal_(out, 0.0, s, -2 * s, 2 * s, generator=gen)
    return init


def _cls(java, fn):
    return type(java, (IWeightInit,), {"JAVA": java, "init": fn})


WeightInitXavier = _cls("WeightInitXavier", _normal(lambda i, o: math.sqrt(2.0 / (i + o))))
WeightInitXavierUniform = _cls("WeightInitXavierUniform", _uniform(lambda i, o: math.sqrt(6.0 / (i + o))))
WeightInitXavierFanIn = _cls("WeightInitXavierFanIn", _normal(lambda i, o: math.sqrt(1.0 / i)))
WeightInitXavierLegacy = _cls("WeightInitXavierLegacy", _normal(lambda i, o: math.sqrt(1.0 / (i + o))))
WeightInitRelu = _cls("WeightInitRelu", _normal(lambda i, o: math.sqrt(2.0 / i)))
WeightInitReluUniform = _cls("WeightInitReluUniform", _uniform(lambda i, o: math.sqrt(6.0 / i)))
WeightInitSigmoidUniform = _cls("WeightInitSigmoidUniform", _uniform(lambda i, o: 4.0 * math.sqrt(6.0 / (i + o))))
WeightInitLecunNormal = _cls("WeightInitLecunNormal", _normal(lambda i, o: math.sqrt(1.0 / i)))
WeightInitLecunUniform = _cls("WeightInitLecunUniform", _uniform(lambda i, o: 3.0 / math.sqrt(i)))
WeightInitNormal = _cls("WeightInitNormal", _normal(lambda i, o: 1.0 / math.sqrt(i)))
WeightInitUniform = _cls("WeightInitUniform", _uniform(lambda i, o: 1.0 / math.sqrt(i)))
WeightInitVarScalingNormalFanIn = _cls("WeightInitVarScalingNormalFanIn", _trunc(lambda i, o: math.sqrt(1.0 / i)))
WeightInitVarScalingNormalFanOut = _cls("WeightInitVarScalingNormalFanOut", _trunc(lambda i, o: math.sqrt(1.0 / o)))
WeightInitVarScalingNormalFanAvg = _cls("WeightInitVarScalingNormalFanAvg", _trunc(lambda i, o: math.sqrt(2.0 / (i + o))))
WeightInitVarScalingUniformFanIn = _cls("WeightInitVarScalingUniformFanIn", _uniform(lambda i, o: math.sqrt(3.0 / i)))
WeightInitVarScalingUniformFanOut = _cls("WeightInitVarScalingUniformFanOut", _uniform(lambda i, o: math.sqrt(3.0 / o)))
WeightInitVarScalingUniformFanAvg = _cls("WeightInitVarScalingUniformFanAvg", _uniform(lambda i, o: math.sqrt(6.0 / (i + o))))
WeightInitConstant = None  # defined below


class WeightInitZero(IWeightInit):
    JAVA = "WeightInitConstant"
    def __init__(self, value=0.0): self.value = float(value)
    def init(self, fanIn, fanOut, out, gen=None): out.fill_(self.value)
    def to_json(self): return {"@class": _PKG + self.JAVA, "value": self.value}


WeightInitConstant = WeightInitZero


class WeightInitIdentity(IWeightInit):
    JAVA = "WeightInitIdentity"
    def __init__(self, scale=None): self.scale = scale
    def init(self, fanIn, fanOut, out, gen=None):
        out.zero_()
        if out.dim() == 2:
            n = min(out.shape)
            out[torch.arange(n), torch.arange(n)] = 1.0 if self.scale is None else self.scale
        else:  # conv kernels [out, in, kh, kw...]: identity at the spatial centre
            centre = tuple(s // 2 for s in out.shape[2:])
            for i in range(min(out.shape[0], out.shape[1])):
                out[(i, i) + centre] = 1.0 if self.scale is None else self.scale
    def to_json(self): return {"@class": _PKG + self.JAVA, "scale": self.scale}


class WeightInitDistribution(IWeightInit):
    JAVA = "WeightInitDistribution"
    def __init__(self, distribution): self.distribution = distribution
    def init(self, fanIn, fanOut, out, gen=None): self.distribution.sample_(out, gen)
    def to_json(self): return {"@class": _PKG + self.JAVA, "distribution": self.distribution.to_json()}


class WeightInit:
    """``org.deeplearning4j.nn.weights.WeightInit`` enum."""
    DISTRIBUTION = "DISTRIBUTION"; ZERO = "ZERO"; ONES = "ONES"; SIGMOID_UNIFORM = "SIGMOID_UNIFORM"
    NORMAL = "NORMAL"; LECUN_NORMAL = "LECUN_NORMAL"; UNIFORM = "UNIFORM"; XAVIER = "XAVIER"
    XAVIER_UNIFORM = "XAVIER_UNIFORM"; XAVIER_FAN_IN = "XAVIER_FAN_IN"; XAVIER_LEGACY = "XAVIER_LEGACY"
    RELU = "RELU"; RELU_UNIFORM = "RELU_UNIFORM"; IDENTITY = "IDENTITY"; LECUN_UNIFORM = "LECUN_UNIFORM"
    VAR_SCALING_NORMAL_FAN_IN = "VAR_SCALING_NORMAL_FAN_IN"; VAR_SCALING_NORMAL_FAN_OUT = "VAR_SCALING_NORMAL_FAN_OUT"
    VAR_SCALING_NORMAL_FAN_AVG = "VAR_SCALING_NORMAL_FAN_AVG"; VAR_SCALING_UNIFORM_FAN_IN = "VAR_SCALING_UNIFORM_FAN_IN"
    VAR_SCALING_UNIFORM_FAN_OUT = "VAR_SCALING_UNIFORM_FAN_OUT"; VAR_SCALING_UNIFORM_FAN_AVG = "VAR_SCALING_UNIFORM_FAN_AVG"

    _MAP = {"ZERO": lambda: WeightInitZero(0.0), "ONES": lambda: WeightInitZero(1.0),
            "SIGMOID_UNIFORM": WeightInitSigmoidUniform, "NORMAL": WeightInitNormal,
            "LECUN_NORMAL": WeightInitLecunNormal, "UNIFORM": WeightInitUniform, "XAVIER": WeightInitXavier,
            "XAVIER_UNIFORM": WeightInitXavierUniform, "XAVIER_FAN_IN": WeightInitXavierFanIn,
            "XAVIER_LEGACY": WeightInitXavierLegacy, "RELU": WeightInitRelu, "RELU_UNIFORM": WeightInitReluUniform,
            "IDENTITY": WeightInitIdentity, "LECUN_UNIFORM": WeightInitLecunUniform,
            "VAR_SCALING_NORMAL_FAN_IN": WeightInitVarScalingNormalFanIn,
            "VAR_SCALING_NORMAL_FAN_OUT": WeightInitVarScalingNormalFanOut,
            "VAR_SCALING_NORMAL_FAN_AVG": WeightInitVarScalingNormalFanAvg,
            "VAR_SCALING_UNIFORM_FAN_IN": WeightInitVarScalingUniformFanIn,
            "VAR_SCALING_UNIFORM_FAN_OUT": WeightInitVarScalingUniformFanOut,
            "VAR_SCALING_UNIFORM_FAN_AVG": WeightInitVarScalingUniformFanAvg}

    @staticmethod
    def get(w, distribution=None) -> IWeightInit:
        if isinstance(w, IWeightInit):
            return w
        if isinstance(w, Distribution):
            return WeightInitDistribution(w)
        if w is None:
            return WeightInitXavier()
        w = str(w).upper()
        if w == "DISTRIBUTION":
            return WeightInitDistribution(distribution)
        return WeightInit._MAP[w]()

    @staticmethod
    def from_json(d):
        if d is None:
            return None
        if isinstance(d, str):
            return WeightInit.get(d)
        name = d["@class"].rsplit(".", 1)[-1]
        if name == "WeightInitConstant":
            return WeightInitZero(d.get("value", 0.0))
        if name == "WeightInitIdentity":
            return WeightInitIdentity(d.get("scale"))
        if name == "WeightInitDistribution":
            return WeightInitDistribution(distribution_from_json(d["distribution"]))
        for f in WeightInit._MAP.values():
            o = f()
            if o.JAVA == name:
                return o
        raise ValueError(f"unknown weight init {name}")
