"""Activation functions (``org.nd4j.linalg.activations.impl.*``, 22 classes).

Each activation is a config object with a ``@class`` id for JSON and a differentiable torch
``__call__``.  Backward comes from autograd; the formulas follow the reference's op
definitions (e.g. rational tanh ``1.7159*tanh_approx(2x/3)``,
``libnd4j/include/ops/ops.h`` functors; hard sigmoid ``clip(0.2x+0.5,0,1)``).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

_PKG = "org.nd4j.linalg.activations.impl."


class IActivation:
    JAVA_CLASS = ""
    NAME = ""
    FIELDS: tuple = ()

    def __call__(self, x: torch.Tensor, training: bool = False) -> torch.Tensor:
        raise NotImplementedError

    def to_json(self):
        d = {"@class": self.JAVA_CLASS}
        for f in self.FIELDS:
            d[f] = getattr(self, f)
        return d

    def __eq__(self, o):
        return type(self) is type(o) and all(getattr(self, f) == getattr(o, f) for f in self.FIELDS)

    def __hash__(self):
        return hash(type(self))

    def __repr__(self):
        return self.NAME


def _mk(name, java, fn, fields=(), defaults=None):
    defaults = defaults or {}

    def __init__(self, *a, **kw):
        for i, f in enumerate(fields):
            setattr(self, f, a[i] if i < len(a) else kw.get(f, defaults.get(f)))

    cls = type("Activation" + java, (IActivation,), {
        "JAVA_CLASS": _PKG + "Activation" + java, "NAME": name, "FIELDS": tuple(fields),
        "__init__": __init__, "__call__": fn})
    return cls


def _rational_tanh(self, x, training=False):
    # 1.7159 * tanh(2x/3) with tanh(y) ~ sgn(y) * (1 - 1/(1+|y|+y^2+1.41645*y^4))
    y = x * (2.0 / 3.0)
    a = y.abs()
    return 1.7159 * torch.sign(y) * (1.0 - 1.0 / (1.0 + a + y * y + 1.41645 * (y ** 4)))


def _rrelu(self, x, training=False):
    if training:
        return F.rrelu(x, self.l, self.u, training=True)
    return F.leaky_relu(x, (self.l + self.u) / 2.0)


ActivationCube = _mk("cube", "Cube", lambda s, x, training=False: x * x * x)
ActivationELU = _mk("elu", "ELU", lambda s, x, training=False: F.elu(x, s.alpha), ("alpha",), {"alpha": 1.0})
ActivationGELU = _mk("gelu", "GELU",
                     lambda s, x, training=False: F.gelu(x, approximate="tanh") if s.precise else x * torch.sigmoid(1.702 * x),
                     ("precise",), {"precise": False})
ActivationHardSigmoid = _mk("hardsigmoid", "HardSigmoid",
                            lambda s, x, training=False: torch.clamp(0.2 * x + 0.5, 0.0, 1.0))
ActivationHardTanH = _mk("hardtanh", "HardTanH", lambda s, x, training=False: F.hardtanh(x))
ActivationIdentity = _mk("identity", "Identity", lambda s, x, training=False: x)
ActivationLReLU = _mk("leakyrelu", "LReLU", lambda s, x, training=False: F.leaky_relu(x, s.alpha),
                      ("alpha",), {"alpha": 0.01})
ActivationMish = _mk("mish", "Mish", lambda s, x, training=False: F.mish(x))
ActivationRReLU = _mk("rrelu", "RReLU", _rrelu, ("l", "u"), {"l": 1.0 / 8, "u": 1.0 / 3})
ActivationRationalTanh = _mk("rationaltanh", "RationalTanh", _rational_tanh)
ActivationReLU = _mk("relu", "ReLU",
                     lambda s, x, training=False: F.relu(x) if s.max is None and not s.threshold and not s.negativeSlope
                     else _relu_general(x, s.max, s.threshold or 0.0, s.negativeSlope or 0.0),
                     ("max", "threshold", "negativeSlope"), {})
ActivationReLU6 = _mk("relu6", "ReLU6", lambda s, x, training=False: F.relu6(x))
ActivationRectifiedTanh = _mk("rectifiedtanh", "RectifiedTanh", lambda s, x, training=False: F.relu(torch.tanh(x)))
ActivationSELU = _mk("selu", "SELU", lambda s, x, training=False: F.selu(x))
ActivationSigmoid = _mk("sigmoid", "Sigmoid", lambda s, x, training=False: torch.sigmoid(x))
ActivationSoftPlus = _mk("softplus", "SoftPlus", lambda s, x, training=False: F.softplus(x))
ActivationSoftSign = _mk("softsign", "SoftSign", lambda s, x, training=False: F.softsign(x))
ActivationSoftmax = _mk("softmax", "Softmax", lambda s, x, training=False: torch.softmax(x, dim=-1 if x.dim() != 3 else 1))
ActivationSwish = _mk("swish", "Swish", lambda s, x, training=False: F.silu(x))
ActivationTanH = _mk("tanh", "TanH", lambda s, x, training=False: torch.tanh(x))
ActivationThresholdedReLU = _mk("thresholdedrelu", "ThresholdedReLU",
                                lambda s, x, training=False: torch.where(x > s.theta, x, torch.zeros_like(x)),
                                ("theta",), {"theta": 1.0})


class ActivationPReLU(IActivation):
    """Parametric ReLU with a learned ``alpha`` array (``ActivationPReLU.java``)."""
    JAVA_CLASS = _PKG + "ActivationPReLU"
    NAME = "prelu"
    FIELDS = ("sharedAxes",)

    def __init__(self, alpha=None, sharedAxes=None):
        self.alpha, self.sharedAxes = alpha, sharedAxes

    def __call__(self, x, training=False):
        return torch.where(x >= 0, x, x * self.alpha)


def _relu_general(x, mx, thr, slope):
    y = torch.where(x > thr, x, slope * (x - thr) if slope else torch.zeros_like(x))
    if mx is not None:
        y = torch.clamp_max(y, mx)
    return y


class Activation:
    """``org.nd4j.linalg.activations.Activation`` enum."""
    CUBE = "CUBE"; ELU = "ELU"; HARDSIGMOID = "HARDSIGMOID"; HARDTANH = "HARDTANH"; IDENTITY = "IDENTITY"
    LEAKYRELU = "LEAKYRELU"; RATIONALTANH = "RATIONALTANH"; RELU = "RELU"; RELU6 = "RELU6"; RRELU = "RRELU"
    SIGMOID = "SIGMOID"; SOFTMAX = "SOFTMAX"; SOFTPLUS = "SOFTPLUS"; SOFTSIGN = "SOFTSIGN"; TANH = "TANH"
    RECTIFIEDTANH = "RECTIFIEDTANH"; SELU = "SELU"; SWISH = "SWISH"; THRESHOLDEDRELU = "THRESHOLDEDRELU"
    GELU = "GELU"; MISH = "MISH"

    _MAP = {"CUBE": ActivationCube, "ELU": ActivationELU, "HARDSIGMOID": ActivationHardSigmoid,
            "HARDTANH": ActivationHardTanH, "IDENTITY": ActivationIdentity, "LEAKYRELU": ActivationLReLU,
            "RATIONALTANH": ActivationRationalTanh, "RELU": ActivationReLU, "RELU6": ActivationReLU6,
            "RRELU": ActivationRReLU, "SIGMOID": ActivationSigmoid, "SOFTMAX": ActivationSoftmax,
            "SOFTPLUS": ActivationSoftPlus, "SOFTSIGN": ActivationSoftSign, "TANH": ActivationTanH,
            "RECTIFIEDTANH": ActivationRectifiedTanh, "SELU": ActivationSELU, "SWISH": ActivationSwish,
            "THRESHOLDEDRELU": ActivationThresholdedReLU, "GELU": ActivationGELU, "MISH": ActivationMish}

    @staticmethod
    def get(a) -> IActivation:
        if isinstance(a, IActivation):
            return a
        if a is None:
            return ActivationIdentity()
        return Activation._MAP[str(a).upper()]()

    @staticmethod
    def from_json(d) -> IActivation:
        if d is None:
            return None
        if isinstance(d, str):
            return Activation.get(d)
        cls_name = d["@class"].rsplit(".", 1)[-1]
        for c in list(Activation._MAP.values()) + [ActivationPReLU]:
            if c.JAVA_CLASS.endswith("." + cls_name):
                obj = c.__new__(c)
                for f in c.FIELDS:
                    setattr(obj, f, d.get(f))
                if c is ActivationPReLU:
                    obj.alpha = None
                return obj
        raise ValueError(f"unknown activation {d['@class']}")
