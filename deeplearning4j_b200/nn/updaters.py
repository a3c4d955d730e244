"""Updater configs (``IUpdater``), their stateful appliers (``GradientUpdater``), learning-rate
schedules (``ISchedule``) and regularizers.

Formulas are those of the native updater helpers
(``libnd4j/include/ops/declarable/helpers/cpu/updater*.cpp`` and ``cuda/updater*.cu``), state
layouts those of the Java updaters (``nd4j-api/.../linalg/learning/*Updater.java``; e.g. Adam
``[M|V]`` halves ``AdamUpdater.java:76-95``, AMSGrad ``[M|V|Vhat]``, AdaDelta ``[msg|msdx]``).

``apply(grad, state, lr, iteration)`` turns the gradient view into the *update* in place; the
caller then subtracts it from the parameters.  The fused CUDA path (one launch over the whole
flattened buffer) lives in ``ops.fused`` and is selected by the networks when the buffers are
on a GPU; these torch versions are the oracle and the CPU path.
"""
from __future__ import annotations

import math

import torch

_CFG = "org.nd4j.linalg.learning.config."
_SCH = "org.nd4j.linalg.schedule."
_REG = "org.nd4j.linalg.learning.regularization."


# --------------------------------------------------------------------------- schedules
class ScheduleType:
    ITERATION = "ITERATION"
    EPOCH = "EPOCH"


class ISchedule:
    JAVA = ""
    FIELDS: tuple = ()

    def valueAt(self, iteration: int, epoch: int) -> float:
        raise NotImplementedError

    def _i(self, iteration, epoch):
        return iteration if self.scheduleType == ScheduleType.ITERATION else epoch

    def to_json(self):
        d = {"@class": _SCH + self.JAVA}
        for f in self.FIELDS:
            d[f] = getattr(self, f)
        return d

    def __eq__(self, o):
        return type(self) is type(o) and self.to_json() == o.to_json()

    def __hash__(self):
        return hash(type(self))


class FixedSchedule(ISchedule):
    JAVA = "FixedSchedule"; FIELDS = ("value",)
    def __init__(self, value): self.value = float(value)
    def valueAt(self, iteration, epoch): return self.value


class ExponentialSchedule(ISchedule):
    JAVA = "ExponentialSchedule"; FIELDS = ("scheduleType", "initialValue", "gamma")
    def __init__(self, scheduleType, initialValue, gamma):
        self.scheduleType, self.initialValue, self.gamma = scheduleType, float(initialValue), float(gamma)
    def valueAt(self, iteration, epoch): return self.initialValue * math.pow(self.gamma, self._i(iteration, epoch))


class InverseSchedule(ISchedule):
    JAVA = "InverseSchedule"; FIELDS = ("scheduleType", "initialValue", "gamma", "power")
    def __init__(self, scheduleType, initialValue, gamma, power):
        self.scheduleType, self.initialValue, self.gamma, self.power = scheduleType, float(initialValue), float(gamma), float(power)
    def valueAt(self, iteration, epoch):
        return self.initialValue / math.pow(1 + self.gamma * self._i(iteration, epoch), self.power)


class MapSchedule(ISchedule):
    JAVA = "MapSchedule"; FIELDS = ("scheduleType", "values")
    def __init__(self, scheduleType, values):
        self.scheduleType = scheduleType
        self.values = {int(k): float(v) for k, v in values.items()}
        if 0 not in self.values:
            raise ValueError("MapSchedule needs a value for position 0")
    def valueAt(self, iteration, epoch):
        i = self._i(iteration, epoch)
        key = max(k for k in self.values if k <= i)
        return self.values[key]
    def to_json(self):
        return {"@class": _SCH + self.JAVA, "scheduleType": self.scheduleType,
                "values": {str(k): v for k, v in sorted(self.values.items())}}


class PolySchedule(ISchedule):
    JAVA = "PolySchedule"; FIELDS = ("scheduleType", "initialValue", "power", "maxIter")
    def __init__(self, scheduleType, initialValue, power, maxIter):
        self.scheduleType, self.initialValue, self.power, self.maxIter = scheduleType, float(initialValue), float(power), int(maxIter)
    def valueAt(self, iteration, epoch):
        return self.initialValue * math.pow(1 + self._i(iteration, epoch) / self.maxIter, -self.power)


class SigmoidSchedule(ISchedule):
    JAVA = "SigmoidSchedule"; FIELDS = ("scheduleType", "initialValue", "gamma", "stepSize")
    def __init__(self, scheduleType, initialValue, gamma, stepSize):
        self.scheduleType, self.initialValue, self.gamma, self.stepSize = scheduleType, float(initialValue), float(gamma), int(stepSize)
    def valueAt(self, iteration, epoch):
        return self.initialValue / (1.0 + math.exp(-self.gamma * (self._i(iteration, epoch) - self.stepSize)))


class StepSchedule(ISchedule):
    JAVA = "StepSchedule"; FIELDS = ("scheduleType", "initialValue", "decayRate", "step")
    def __init__(self, scheduleType, initialValue, decayRate, step):
        self.scheduleType, self.initialValue, self.decayRate, self.step = scheduleType, float(initialValue), float(decayRate), float(step)
    def valueAt(self, iteration, epoch):
        return self.initialValue * math.pow(self.decayRate, math.floor(self._i(iteration, epoch) / self.step))


class RampSchedule(ISchedule):
    """Linear warm-up over ``numIter`` iterations wrapped around a base schedule."""
    JAVA = "RampSchedule"; FIELDS = ("baseSchedule", "numIter")
    def __init__(self, baseSchedule, numIter):
        self.baseSchedule, self.numIter = baseSchedule, int(numIter)
    def valueAt(self, iteration, epoch):
        base = self.baseSchedule.valueAt(iteration, epoch)
        if iteration >= self.numIter - 1:
            return base
        return base * (iteration + 1) / self.numIter
    def to_json(self):
        return {"@class": _SCH + self.JAVA, "baseSchedule": self.baseSchedule.to_json(), "numIter": self.numIter}


class CycleSchedule(ISchedule):
    """1-cycle schedule: ramp up, ramp down, then anneal (``CycleSchedule.java``)."""
    JAVA = "CycleSchedule"
    FIELDS = ("scheduleType", "initialLearningRate", "maxLearningRate", "cycleLength", "annealingLength", "annealingDecay")
    def __init__(self, scheduleType, initialLearningRate=None, maxLearningRate=0.1, cycleLength=100, annealingLength=None, annealingDecay=0.1):
        self.scheduleType = scheduleType
        self.maxLearningRate = float(maxLearningRate)
        self.initialLearningRate = float(initialLearningRate if initialLearningRate is not None else maxLearningRate * 0.1)
        self.cycleLength = int(cycleLength)
        self.annealingLength = int(annealingLength if annealingLength is not None else round(cycleLength * 0.1))
        self.annealingDecay = float(annealingDecay)
        self.stepSize = (self.cycleLength - self.annealingLength) // 2
        self.increment = (self.maxLearningRate - self.initialLearningRate) / self.stepSize
    def valueAt(self, iteration, epoch):
        pos = self._i(iteration, epoch) % self.cycleLength
        if pos < self.stepSize:
            return self.initialLearningRate + self.increment * pos
        if pos < 2 * self.stepSize:
            return self.maxLearningRate - self.increment * (pos - self.stepSize)
        return self.initialLearningRate * math.pow(self.annealingDecay, self.annealingLength - (self.cycleLength - pos))


SCHEDULES = {c.JAVA: c for c in (FixedSchedule, ExponentialSchedule, InverseSchedule, MapSchedule, PolySchedule,
                                 SigmoidSchedule, StepSchedule, RampSchedule, CycleSchedule)}


def schedule_from_json(d):
    if d is None:
        return None
    cls = SCHEDULES[d["@class"].rsplit(".", 1)[-1]]
    kw = {k: v for k, v in d.items() if k != "@class"}
    if cls is RampSchedule:
        kw["baseSchedule"] = schedule_from_json(kw["baseSchedule"])
    if cls is CycleSchedule:
        kw.pop("stepSize", None); kw.pop("increment", None)
    return cls(**kw)


# --------------------------------------------------------------------------- regularization
class Regularization:
    JAVA = ""
    APPLY_STEP = "BEFORE_UPDATER"

    def __init__(self, coeff):
        self.coeff = coeff  # float or ISchedule

    def value(self, iteration, epoch):
        return self.coeff.valueAt(iteration, epoch) if isinstance(self.coeff, ISchedule) else float(self.coeff)

    def __eq__(self, o):
        return type(self) is type(o) and self.to_json() == o.to_json()

    def __hash__(self):
        return hash(type(self))


class L1Regularization(Regularization):
    JAVA = "L1Regularization"
    def apply(self, param, grad, lr, iteration, epoch):
        grad.add_(torch.sign(param), alpha=self.value(iteration, epoch))
    def score(self, param, iteration, epoch):
        return self.value(iteration, epoch) * param.abs().sum()
    def to_json(self):
        return {"@class": _REG + self.JAVA, "l1": _sched_or_value(self.coeff)}


class L2Regularization(Regularization):
    JAVA = "L2Regularization"
    def apply(self, param, grad, lr, iteration, epoch):
        grad.add_(param, alpha=self.value(iteration, epoch))
    def score(self, param, iteration, epoch):
        return 0.5 * self.value(iteration, epoch) * (param * param).sum()
    def to_json(self):
        return {"@class": _REG + self.JAVA, "l2": _sched_or_value(self.coeff)}


class WeightDecay(Regularization):
    """``update += coeff * (lr if applyLR else 1) * param`` after the updater (``WeightDecay.java``)."""
    JAVA = "WeightDecay"
    APPLY_STEP = "POST_UPDATER"
    def __init__(self, coeff, applyLR=True):
        super().__init__(coeff)
        self.applyLR = applyLR
    def apply(self, param, grad, lr, iteration, epoch):
        c = self.value(iteration, epoch) * (lr if self.applyLR else 1.0)
        grad.add_(param, alpha=c)
    def score(self, param, iteration, epoch):
        return 0.5 * self.value(iteration, epoch) * (param * param).sum()
    def to_json(self):
        return {"@class": _REG + self.JAVA, "applyLR": self.applyLR, "coeff": _sched_or_value(self.coeff)}


def _sched_or_value(v):
    if isinstance(v, ISchedule):
        return v.to_json()
    return {"@class": _SCH + "FixedSchedule", "value": float(v)}


def regularization_from_json(d):
    name = d["@class"].rsplit(".", 1)[-1]
    def val(x):
        if isinstance(x, dict):
            s = schedule_from_json(x)
            return s.value if isinstance(s, FixedSchedule) else s
        return x
    if name == "L1Regularization":
        return L1Regularization(val(d["l1"]))
    if name == "L2Regularization":
        return L2Regularization(val(d["l2"]))
    return WeightDecay(val(d["coeff"]), d.get("applyLR", True))


# --------------------------------------------------------------------------- updaters
class IUpdater:
    JAVA = ""
    FIELDS: tuple = ()
    STATE_MULT = 0   # state elements per parameter
    KERNEL_ID = -1   # id understood by the fused CUDA updater kernel

    learningRate = 0.0
    learningRateSchedule = None

    def stateSize(self, numParams: int) -> int:
        return self.STATE_MULT * numParams

    def hasLearningRate(self):
        return True

    def getLearningRate(self, iteration: int, epoch: int) -> float:
        if self.learningRateSchedule is not None:
            return self.learningRateSchedule.valueAt(iteration, epoch)
        return self.learningRate

    def setLrAndSchedule(self, lr, schedule):
        self.learningRate, self.learningRateSchedule = lr, schedule

    def clone(self):
        import copy
        return copy.deepcopy(self)

    def instantiate(self, state_view, initialize=True):
        return GradientUpdater(self, state_view, initialize)

    def apply(self, g, state, lr, t):
        raise NotImplementedError

    def to_json(self):
        d = {"@class": _CFG + self.JAVA}
        for f in self.FIELDS:
            v = getattr(self, f)
            d[f] = v.to_json() if isinstance(v, ISchedule) else v
        return d

    def __eq__(self, o):
        return type(self) is type(o) and self.to_json() == o.to_json()

    def __hash__(self):
        return hash((type(self), self.learningRate))

    def __repr__(self):
        return f"{self.JAVA}({', '.join(f'{f}={getattr(self, f)}' for f in self.FIELDS)})"


def _lr_args(lr, default):
    if isinstance(lr, ISchedule):
        return default, lr
    return (default if lr is None else float(lr)), None


def _eps_t(lr, b1, b2, t, eps, with_sqrt=True):
    b1t = 1.0 - b1 ** (t + 1)
    num = lr * (math.sqrt(1.0 - b2 ** (t + 1)) if with_sqrt else 1.0)
    e = num / b1t if b1t != 0 else float("nan")
    if math.isnan(e) or e == 0.0 or math.isinf(e):
        e = eps
    return e


class Sgd(IUpdater):
    JAVA = "Sgd"; FIELDS = ("learningRate", "learningRateSchedule"); STATE_MULT = 0; KERNEL_ID = 0
    def __init__(self, learningRate=None):
        self.learningRate, self.learningRateSchedule = _lr_args(learningRate, 1e-3)
    def apply(self, g, state, lr, t):
        g.mul_(lr)


class NoOp(IUpdater):
    JAVA = "NoOp"; FIELDS = (); STATE_MULT = 0; KERNEL_ID = 9
    def hasLearningRate(self): return False
    def apply(self, g, state, lr, t): pass


class Nesterovs(IUpdater):
    JAVA = "Nesterovs"; FIELDS = ("learningRate", "learningRateSchedule", "momentum", "momentumISchedule")
    STATE_MULT = 1; KERNEL_ID = 1
    def __init__(self, learningRate=None, momentum=0.9, momentumSchedule=None):
        self.learningRate, self.learningRateSchedule = _lr_args(learningRate, 0.1)
        self.momentum, self.momentumISchedule = float(momentum), momentumSchedule
    def currentMomentum(self, iteration, epoch):
        return self.momentumISchedule.valueAt(iteration, epoch) if self.momentumISchedule else self.momentum
    def apply(self, g, state, lr, t, momentum=None):
        mu = self.momentum if momentum is None else momentum
        v = state
        prev = v * mu                       # vPrev = mu * v
        torch.sub(prev, g, alpha=lr, out=v)  # v = vPrev - lr*g
        torch.add(prev, v, alpha=(-mu - 1.0), out=g)  # update = vPrev - (1+mu) v


class Adam(IUpdater):
    JAVA = "Adam"; FIELDS = ("beta1", "beta2", "epsilon", "learningRate", "learningRateSchedule")
    STATE_MULT = 2; KERNEL_ID = 2
    def __init__(self, learningRate=None, beta1=0.9, beta2=0.999, epsilon=1e-8):
        self.learningRate, self.learningRateSchedule = _lr_args(learningRate, 1e-3)
        self.beta1, self.beta2, self.epsilon = float(beta1), float(beta2), float(epsilon)
    def apply(self, g, state, lr, t):
        n = g.numel()
        m, v = state[:n].view_as(g), state[n:2 * n].view_as(g)
        m.mul_(self.beta1).add_(g, alpha=1 - self.beta1)
        v.mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
        e = _eps_t(lr, self.beta1, self.beta2, t, self.epsilon)
        torch.div(m * e, v.sqrt().add_(self.epsilon), out=g)


class AdaMax(Adam):
    JAVA = "AdaMax"; KERNEL_ID = 3
    def apply(self, g, state, lr, t):
        n = g.numel()
        m, u = state[:n].view_as(g), state[n:2 * n].view_as(g)
        m.mul_(self.beta1).add_(g, alpha=1 - self.beta1)
        torch.maximum(u * self.beta2, g.abs(), out=u)
        u.add_(1e-32)
        e = _eps_t(lr, self.beta1, self.beta2, t, self.epsilon, with_sqrt=False)
        torch.div(m * e, u, out=g)


class Nadam(Adam):
    JAVA = "Nadam"; KERNEL_ID = 4
    def apply(self, g, state, lr, t):
        n = g.numel()
        m, v = state[:n].view_as(g), state[n:2 * n].view_as(g)
        omb1g = g * (1 - self.beta1)
        m.mul_(self.beta1).add_(omb1g)
        v.mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
        mb1t = 1.0 - self.beta1 ** (t + 1)
        torch.div(lr * ((m * self.beta1 + omb1g) / mb1t), v.sqrt().add_(self.epsilon), out=g)


class AMSGrad(Adam):
    JAVA = "AMSGrad"; STATE_MULT = 3; KERNEL_ID = 5
    def apply(self, g, state, lr, t):
        n = g.numel()
        m, v, h = state[:n].view_as(g), state[n:2 * n].view_as(g), state[2 * n:3 * n].view_as(g)
        m.mul_(self.beta1).add_(g, alpha=1 - self.beta1)
        v.mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
        torch.maximum(h, v, out=h)
        e = _eps_t(lr, self.beta1, self.beta2, t, self.epsilon)
        torch.div(m * e, h.sqrt().add_(self.epsilon), out=g)


class AdaBelief(Adam):
    JAVA = "AdaBelief"; KERNEL_ID = 6
    def __init__(self, learningRate=None, beta1=0.9, beta2=0.999, epsilon=1e-14):
        super().__init__(learningRate, beta1, beta2, epsilon)
    def apply(self, g, state, lr, t):
        n = g.numel()
        m, s = state[:n].view_as(g), state[n:2 * n].view_as(g)
        m.mul_(self.beta1).add_(g, alpha=1 - self.beta1)
        d = g - m
        s.mul_(self.beta2).addcmul_(d, d, value=1 - self.beta2).add_(self.epsilon)
        e = _eps_t(lr, self.beta1, self.beta2, t, self.epsilon)
        torch.div(m * e, s.sqrt().add_(self.epsilon), out=g)


class AdaGrad(IUpdater):
    JAVA = "AdaGrad"; FIELDS = ("epsilon", "learningRate", "learningRateSchedule"); STATE_MULT = 1; KERNEL_ID = 7
    def __init__(self, learningRate=None, epsilon=1e-6):
        self.learningRate, self.learningRateSchedule = _lr_args(learningRate, 1e-1)
        self.epsilon = float(epsilon)
    def apply(self, g, state, lr, t):
        h = state.view_as(g)
        h.addcmul_(g, g)
        torch.div(g * lr, h.sqrt().add_(self.epsilon), out=g)


class RmsProp(IUpdater):
    JAVA = "RmsProp"; FIELDS = ("epsilon", "learningRate", "learningRateSchedule", "rmsDecay"); STATE_MULT = 1; KERNEL_ID = 8
    def __init__(self, learningRate=None, rmsDecay=0.95, epsilon=1e-8):
        self.learningRate, self.learningRateSchedule = _lr_args(learningRate, 1e-1)
        self.rmsDecay, self.epsilon = float(rmsDecay), float(epsilon)
    def apply(self, g, state, lr, t):
        s = state.view_as(g)
        s.mul_(self.rmsDecay).addcmul_(g, g, value=1 - self.rmsDecay)
        torch.div(g * lr, s.sqrt().add_(self.epsilon), out=g)


class AdaDelta(IUpdater):
    JAVA = "AdaDelta"; FIELDS = ("epsilon", "rho"); STATE_MULT = 2; KERNEL_ID = 10
    def __init__(self, rho=0.95, epsilon=1e-6):
        self.rho, self.epsilon = float(rho), float(epsilon)
    def hasLearningRate(self): return False
    def apply(self, g, state, lr, t):
        n = g.numel()
        msg, msdx = state[:n].view_as(g), state[n:2 * n].view_as(g)
        msg.mul_(self.rho).addcmul_(g, g, value=1 - self.rho)
        up = g * ((msdx + self.epsilon).sqrt() / (msg + self.epsilon).sqrt())
        msdx.mul_(self.rho).addcmul_(up, up, value=1 - self.rho)
        g.copy_(up)


UPDATERS = {c.JAVA: c for c in (Sgd, NoOp, Nesterovs, Adam, AdaMax, Nadam, AMSGrad, AdaBelief, AdaGrad, RmsProp, AdaDelta)}


def updater_from_json(d):
    if d is None:
        return None
    cls = UPDATERS[d["@class"].rsplit(".", 1)[-1]]
    obj = cls.__new__(cls)
    for f in cls.FIELDS:
        v = d.get(f)
        if f in ("learningRateSchedule", "momentumISchedule"):
            v = schedule_from_json(v)
        setattr(obj, f, v)
    return obj


class GradientUpdater:
    """Stateful applier bound to a view of the flat updater-state buffer."""

    def __init__(self, config: IUpdater, state_view, initialize=True):
        self.config = config
        self.state = state_view
        if initialize and state_view is not None and state_view.numel():
            state_view.zero_()

    def setStateViewArray(self, view, initialize=False):
        self.state = view
        if initialize:
            view.zero_()

    def getState(self):
        return self.state

    def applyUpdater(self, gradient, iteration: int, epoch: int = 0):
        c = self.config
        lr = c.getLearningRate(iteration, epoch) if c.hasLearningRate() else 0.0
        if isinstance(c, Nesterovs):
            c.apply(gradient, self.state.view_as(gradient), lr, iteration, c.currentMomentum(iteration, epoch))
        else:
            c.apply(gradient, self.state, lr, iteration)
        return gradient
