"""Loss functions (``org.nd4j.linalg.lossfunctions.impl.*``, 19 ``ILossFunction`` classes).

``score_array`` returns the per-example loss (``computeScoreArray``); ``score`` reduces it the
way ``ILossFunction.computeScore(labels, preOutput, activationFn, mask, average)`` does.
Gradients w.r.t. the pre-output come from autograd.  The softmax + MCXENT pair is evaluated
through a fused log-softmax (the reference clips the softmax output at ``softmaxClipEps``,
``LossMCXENT.java:97-98``; the fused form is its numerically exact limit).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .activations import Activation, ActivationSoftmax, ActivationSigmoid, IActivation

_PKG = "org.nd4j.linalg.lossfunctions.impl."


def _up(t):
    """At least float32: half / bf16 inputs are computed in fp32, fp64 stays fp64 (gradient checks)."""
    return t if t.dtype in (torch.float32, torch.float64) else t.float()


def _apply_mask(score, mask):
    if mask is None:
        return score
    m = mask
    while m.dim() < score.dim():
        m = m.unsqueeze(-1)
    return score * m.to(score.dtype)


class ILossFunction:
    JAVA_CLASS = ""
    FIELDS: tuple = ()

    def __init__(self, weights=None):
        self.weights = weights

    def name(self):
        return type(self).__name__

    def _elem(self, labels, preout, act: IActivation):
        raise NotImplementedError

    def score_array(self, labels, preout, act, mask=None):
        """Per-example loss, shape [minibatch]."""
        act = Activation.get(act)
        s = self._elem(labels, preout, act)
        if self.weights is not None and s.dim() > 1:
            w = torch.as_tensor(self.weights, dtype=s.dtype, device=s.device)
            s = s * w.reshape([1, -1] + [1] * (s.dim() - 2))
        s = _apply_mask(s, mask)
        if s.dim() > 1:
            s = s.reshape(s.shape[0], -1).sum(1)
        return s

    def score(self, labels, preout, act, mask=None, average=True):
        s = self.score_array(labels, preout, act, mask).sum()
        if average:
            s = s / labels.shape[0]
        return s

    def to_json(self):
        d = {"@class": self.JAVA_CLASS}
        for f in self.FIELDS:
            d[f] = getattr(self, f)
        return d

    def __eq__(self, o):
        return type(self) is type(o)

    def __hash__(self):
        return hash(type(self))


class LossMCXENT(ILossFunction):
    JAVA_CLASS = _PKG + "LossMCXENT"
    FIELDS = ("softmaxClipEps",)

    def __init__(self, weights=None, softmaxClipEps=1e-10):
        super().__init__(weights)
        self.softmaxClipEps = softmaxClipEps

    def _elem(self, labels, preout, act):
        if isinstance(act, ActivationSoftmax):
            dim = 1 if preout.dim() == 3 else -1
            return -(labels * F.log_softmax(_up(preout), dim=dim))
        out = _up(act(preout))
        return -(labels * torch.log(out.clamp(self.softmaxClipEps, 1.0 - self.softmaxClipEps)))


class LossNegativeLogLikelihood(LossMCXENT):
    JAVA_CLASS = _PKG + "LossNegativeLogLikelihood"


class LossSparseMCXENT(LossMCXENT):
    """Labels are class indices ([mb] or [mb,1]) instead of one-hot rows."""
    JAVA_CLASS = _PKG + "LossSparseMCXENT"

    def score_array(self, labels, preout, act, mask=None):
        act = Activation.get(act)
        idx = labels.reshape(labels.shape[0], -1)[:, 0].long() if preout.dim() == 2 else labels.long()
        if isinstance(act, ActivationSoftmax) and preout.dim() == 2:
            s = F.cross_entropy(_up(preout), idx, reduction="none")
        else:
            out = _up(act(preout)).clamp(self.softmaxClipEps, 1 - self.softmaxClipEps)
            s = -torch.log(out.gather(1, idx.reshape(-1, 1))).reshape(-1)
        return _apply_mask(s, mask)


class LossBinaryXENT(ILossFunction):
    JAVA_CLASS = _PKG + "LossBinaryXENT"
    FIELDS = ("clipEps",)

    def __init__(self, weights=None, clipEps=1e-5):
        super().__init__(weights)
        self.clipEps = clipEps

    def _elem(self, labels, preout, act):
        if isinstance(act, ActivationSigmoid):
            return F.binary_cross_entropy_with_logits(_up(preout), _up(labels), reduction="none")
        out = _up(act(preout))
        if self.clipEps:
            out = out.clamp(self.clipEps, 1.0 - self.clipEps)
        return -(labels * torch.log(out) + (1 - labels) * torch.log(1 - out))


class LossMSE(ILossFunction):
    JAVA_CLASS = _PKG + "LossMSE"

    def _elem(self, labels, preout, act):
        d = act(preout) - labels
        return d * d / labels.shape[1]


class LossL2(ILossFunction):
    JAVA_CLASS = _PKG + "LossL2"

    def _elem(self, labels, preout, act):
        d = act(preout) - labels
        return d * d


class LossMAE(ILossFunction):
    JAVA_CLASS = _PKG + "LossMAE"

    def _elem(self, labels, preout, act):
        return (act(preout) - labels).abs() / labels.shape[1]


class LossL1(ILossFunction):
    JAVA_CLASS = _PKG + "LossL1"

    def _elem(self, labels, preout, act):
        return (act(preout) - labels).abs()


class LossMAPE(ILossFunction):
    JAVA_CLASS = _PKG + "LossMAPE"

    def _elem(self, labels, preout, act):
        return 100.0 * ((act(preout) - labels) / labels).abs() / labels.shape[1]


class LossMSLE(ILossFunction):
    JAVA_CLASS = _PKG + "LossMSLE"

    def _elem(self, labels, preout, act):
        d = torch.log((act(preout) + 1.0) / (labels + 1.0))
        return d * d / labels.shape[1]


class LossHinge(ILossFunction):
    JAVA_CLASS = _PKG + "LossHinge"

    def _elem(self, labels, preout, act):
        return torch.clamp_min(1.0 - labels * act(preout), 0.0)


class LossSquaredHinge(ILossFunction):
    JAVA_CLASS = _PKG + "LossSquaredHinge"

    def _elem(self, labels, preout, act):
        h = torch.clamp_min(1.0 - labels * act(preout), 0.0)
        return h * h


class LossKLD(ILossFunction):
    JAVA_CLASS = _PKG + "LossKLD"

    def _elem(self, labels, preout, act):
        out = act(preout).clamp(1e-10, 1.0)
        lab = labels.clamp(1e-10, 1.0)
        return lab * (torch.log(lab) - torch.log(out))


class LossPoisson(ILossFunction):
    JAVA_CLASS = _PKG + "LossPoisson"

    def _elem(self, labels, preout, act):
        out = act(preout)
        return out - labels * torch.log(out.clamp_min(1e-10))


class LossCosineProximity(ILossFunction):
    JAVA_CLASS = _PKG + "LossCosineProximity"

    def score_array(self, labels, preout, act, mask=None):
        out = Activation.get(act)(preout)
        num = (out * labels).reshape(out.shape[0], -1).sum(1)
        den = out.reshape(out.shape[0], -1).norm(dim=1).clamp_min(1e-12) * labels.reshape(out.shape[0], -1).norm(dim=1).clamp_min(1e-12)
        return _apply_mask(-num / den, mask)


class LossWasserstein(ILossFunction):
    JAVA_CLASS = _PKG + "LossWasserstein"

    def _elem(self, labels, preout, act):
        return labels * act(preout) / labels.shape[1]


class LossFMeasure(ILossFunction):
    """Batch-level soft F-beta loss for binary outputs (``LossFMeasure.java``)."""
    JAVA_CLASS = _PKG + "LossFMeasure"
    FIELDS = ("beta",)

    def __init__(self, beta=1.0):
        super().__init__(None)
        self.beta = beta

    def score(self, labels, preout, act, mask=None, average=True):
        out = Activation.get(act)(preout)
        if out.shape[1] == 2:
            out, labels = out[:, 1], labels[:, 1]
        out, labels = out.reshape(-1), labels.reshape(-1)
        if mask is not None:
            out, labels = out * mask.reshape(-1), labels * mask.reshape(-1)
        tp = (out * labels).sum()
        b2 = self.beta ** 2
        num = (1 + b2) * tp
        den = b2 * labels.sum() + out.sum()
        return 1.0 - num / den.clamp_min(1e-12)

    def score_array(self, labels, preout, act, mask=None):
        raise NotImplementedError("LossFMeasure is defined on the whole minibatch only")


class LossMultiLabel(ILossFunction):
    """Pairwise ranking loss over (positive, negative) label pairs (``LossMultiLabel.java``)."""
    JAVA_CLASS = _PKG + "LossMultiLabel"

    def score_array(self, labels, preout, act, mask=None):
        out = Activation.get(act)(preout)
        pos = labels > 0.5
        npos = pos.sum(1).clamp_min(1).to(out.dtype)
        nneg = (~pos).sum(1).clamp_min(1).to(out.dtype)
        diff = out.unsqueeze(2) - out.unsqueeze(1)          # [mb, i, j] = out_i - out_j
        pair = (pos.unsqueeze(2) & (~pos).unsqueeze(1)).to(out.dtype)
        s = (torch.exp(-diff) * pair).sum((1, 2)) / (npos * nneg)
        return _apply_mask(s, mask)


class LossMixtureDensity(ILossFunction):
    """Negative log-likelihood of a Gaussian mixture (``LossMixtureDensity.java``).

    Pre-output layout per example: ``[alpha(k) | sigma(k) | mu(k*labelWidth)]``.
    """
    JAVA_CLASS = _PKG + "LossMixtureDensity"
    FIELDS = ("mixtures", "labelWidth")

    def __init__(self, mixtures=1, labelWidth=1):
        super().__init__(None)
        self.mixtures, self.labelWidth = mixtures, labelWidth

    def score_array(self, labels, preout, act, mask=None):
        k, w = self.mixtures, self.labelWidth
        out = Activation.get(act)(preout)
        log_alpha = F.log_softmax(out[:, :k], dim=1)
        sigma = torch.exp(out[:, k:2 * k])
        mu = out[:, 2 * k:].reshape(-1, k, w)
        d2 = ((labels.unsqueeze(1) - mu) ** 2).sum(2)
        logp = -0.5 * d2 / (sigma * sigma) - w * torch.log(sigma) - 0.5 * w * math.log(2 * math.pi)
        return _apply_mask(-torch.logsumexp(log_alpha + logp, dim=1), mask)


class LossFunctions:
    class LossFunction:
        MSE = "MSE"; L1 = "L1"; XENT = "XENT"; MCXENT = "MCXENT"; SPARSE_MCXENT = "SPARSE_MCXENT"
        SQUARED_LOSS = "SQUARED_LOSS"; RECONSTRUCTION_CROSSENTROPY = "RECONSTRUCTION_CROSSENTROPY"
        NEGATIVELOGLIKELIHOOD = "NEGATIVELOGLIKELIHOOD"; COSINE_PROXIMITY = "COSINE_PROXIMITY"; HINGE = "HINGE"
        SQUARED_HINGE = "SQUARED_HINGE"; KL_DIVERGENCE = "KL_DIVERGENCE"; MEAN_ABSOLUTE_ERROR = "MEAN_ABSOLUTE_ERROR"
        L2 = "L2"; MEAN_ABSOLUTE_PERCENTAGE_ERROR = "MEAN_ABSOLUTE_PERCENTAGE_ERROR"
        MEAN_SQUARED_LOGARITHMIC_ERROR = "MEAN_SQUARED_LOGARITHMIC_ERROR"; POISSON = "POISSON"; WASSERSTEIN = "WASSERSTEIN"

    _MAP = {"MSE": LossMSE, "L1": LossL1, "XENT": LossBinaryXENT, "MCXENT": LossMCXENT,
            "SPARSE_MCXENT": LossSparseMCXENT, "SQUARED_LOSS": LossL2, "RECONSTRUCTION_CROSSENTROPY": LossBinaryXENT,
            "NEGATIVELOGLIKELIHOOD": LossNegativeLogLikelihood, "COSINE_PROXIMITY": LossCosineProximity,
            "HINGE": LossHinge, "SQUARED_HINGE": LossSquaredHinge, "KL_DIVERGENCE": LossKLD,
            "MEAN_ABSOLUTE_ERROR": LossMAE, "L2": LossL2, "MEAN_ABSOLUTE_PERCENTAGE_ERROR": LossMAPE,
            "MEAN_SQUARED_LOGARITHMIC_ERROR": LossMSLE, "POISSON": LossPoisson, "WASSERSTEIN": LossWasserstein}

    ALL = [LossBinaryXENT, LossCosineProximity, LossFMeasure, LossHinge, LossKLD, LossL1, LossL2, LossMAE, LossMAPE,
           LossMCXENT, LossMSE, LossMSLE, LossMixtureDensity, LossMultiLabel, LossNegativeLogLikelihood, LossPoisson,
           LossSparseMCXENT, LossSquaredHinge, LossWasserstein]

    @staticmethod
    def get(l) -> ILossFunction:
        if isinstance(l, ILossFunction):
            return l
        return LossFunctions._MAP[str(l).upper()]()

    @staticmethod
    def from_json(d):
        if d is None:
            return None
        if isinstance(d, str):
            return LossFunctions.get(d)
        name = d["@class"].rsplit(".", 1)[-1]
        for c in LossFunctions.ALL:
            if c.__name__ == name:
                obj = c.__new__(c)
                obj.weights = d.get("weights")
                for f in c.FIELDS:
                    setattr(obj, f, d.get(f))
                return obj
        raise ValueError(f"unknown loss {d['@class']}")
