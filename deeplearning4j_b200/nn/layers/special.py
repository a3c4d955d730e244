"""Less common layers: variational auto-encoder, capsule layers, locally connected layers, the YOLOv2
output layer, the one-class output layer and the user-defined SameDiff layer bases.

Parity: ``nn/conf/layers/variational/*`` + ``nn/layers/variational/VariationalAutoencoder.java``,
``CapsuleLayer.java`` / ``PrimaryCapsules.java`` / ``CapsuleStrengthLayer.java``,
``LocallyConnected1D.java`` / ``LocallyConnected2D.java``, ``objdetect/Yolo2OutputLayer.java``,
``ocnn/OCNNOutputLayer.java`` and ``samediff/{SameDiffLayer,SameDiffLambdaLayer,SameDiffOutputLayer}.java``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ..activations import Activation
from ..conf.base import BaseLayer, FeedForwardLayer, InputType, Layer, NoParamLayer, ParamSpec
from ..losses import ILossFunction, LossFunctions

_L = "org.deeplearning4j.nn.conf.layers."
_V = _L + "variational."


# ============================================================================= reconstruction distributions
class ReconstructionDistribution:
    def distributionInputSize(self, dataSize): return dataSize
    def hasLossFunction(self): return False
    def to_json(self): return {"@class": _V + type(self).__name__}


class GaussianReconstructionDistribution(ReconstructionDistribution):
    """p(x|z) = N(mean, sigma^2); the decoder emits [mean, log(sigma^2)] per input value."""

    def __init__(self, activationFn="identity"):
        self.activationFn = Activation.get(activationFn)

    def distributionInputSize(self, dataSize): return 2 * dataSize

    def _split(self, pre):
        out = self.activationFn(pre, False)
        n = out.shape[1] // 2
        return out[:, :n], out[:, n:]

    def negLogProbability(self, x, pre, average=True):
        mean, log_var = self._split(pre)
        nll = 0.5 * (math.log(2 * math.pi) + log_var + (x - mean) ** 2 / log_var.exp())
        s = nll.sum(1)
        return s.mean() if average else s.sum()

    def exampleNegLogProbability(self, x, pre):
        mean, log_var = self._split(pre)
        return (0.5 * (math.log(2 * math.pi) + log_var + (x - mean) ** 2 / log_var.exp())).sum(1)

    def generateAtMean(self, pre): return self._split(pre)[0]

    def generateRandom(self, pre):
        mean, log_var = self._split(pre)
        return mean + torch.randn_like(mean) * (0.5 * log_var).exp()

    def to_json(self): return {"@class": _V + "GaussianReconstructionDistribution", "activationFn": self.activationFn.to_json()}


class BernoulliReconstructionDistribution(ReconstructionDistribution):
    def __init__(self, activationFn="sigmoid"):
        self.activationFn = Activation.get(activationFn)

    def exampleNegLogProbability(self, x, pre):
        p = self.activationFn(pre, False).clamp(1e-10, 1 - 1e-10)
        return -(x * p.log() + (1 - x) * (1 - p).log()).sum(1)

    def negLogProbability(self, x, pre, average=True):
        s = self.exampleNegLogProbability(x, pre)
        return s.mean() if average else s.sum()

    def generateAtMean(self, pre): return self.activationFn(pre, False)
    def generateRandom(self, pre): return torch.bernoulli(self.activationFn(pre, False))
    def to_json(self): return {"@class": _V + "BernoulliReconstructionDistribution", "activationFn": self.activationFn.to_json()}


class ExponentialReconstructionDistribution(ReconstructionDistribution):
    """p(x|z) = lambda exp(-lambda x) with gamma = log(lambda) emitted by the decoder."""

    def __init__(self, activationFn="identity"):
        self.activationFn = Activation.get(activationFn)

    def exampleNegLogProbability(self, x, pre):
        gamma = self.activationFn(pre, False)
        return -(gamma - x * gamma.exp()).sum(1)

    def negLogProbability(self, x, pre, average=True):
        s = self.exampleNegLogProbability(x, pre)
        return s.mean() if average else s.sum()

    def generateAtMean(self, pre): return (-self.activationFn(pre, False)).exp()

    def generateRandom(self, pre):
        lam = self.activationFn(pre, False).exp()
        return -torch.log(torch.rand_like(lam).clamp_min(1e-12)) / lam

    def to_json(self): return {"@class": _V + "ExponentialReconstructionDistribution", "activationFn": self.activationFn.to_json()}


class LossFunctionWrapper(ReconstructionDistribution):
    """Plain loss function in place of a probabilistic decoder (the layer is then an ordinary auto-encoder)."""

    def __init__(self, activationFn="identity", lossFunction="MSE"):
        self.activationFn = Activation.get(activationFn)
        self.lossFunction = lossFunction if isinstance(lossFunction, ILossFunction) else LossFunctions.get(lossFunction)

    def hasLossFunction(self): return True
    def negLogProbability(self, x, pre, average=True): return self.lossFunction.score(x, pre, self.activationFn, None, average)
    def exampleNegLogProbability(self, x, pre): return self.lossFunction.score_array(x, pre, self.activationFn, None).reshape(x.shape[0], -1).sum(1)
    def generateAtMean(self, pre): return self.activationFn(pre, False)
    generateRandom = generateAtMean

    def to_json(self):
        return {"@class": _V + "LossFunctionWrapper", "activationFn": self.activationFn.to_json(), "lossFunction": self.lossFunction.to_json()}


class CompositeReconstructionDistribution(ReconstructionDistribution):
    """Different distributions for consecutive slices of the data vector."""

    def __init__(self, sizes=None, distributions=None):
        self.sizes, self.distributions = list(sizes or []), list(distributions or [])

    class Builder:
        def __init__(self): self.s, self.d = [], []
        def addDistribution(self, size, dist): self.s.append(int(size)); self.d.append(dist); return self
        def build(self): return CompositeReconstructionDistribution(self.s, self.d)

    def distributionInputSize(self, dataSize): return sum(d.distributionInputSize(s) for s, d in zip(self.sizes, self.distributions))

    def _parts(self, x, pre):
        xo = po = 0
        for s, d in zip(self.sizes, self.distributions):
            ps = d.distributionInputSize(s)
            yield d, (None if x is None else x[:, xo:xo + s]), pre[:, po:po + ps]
            xo, po = xo + s, po + ps

    def exampleNegLogProbability(self, x, pre): return sum(d.exampleNegLogProbability(xs, ps) for d, xs, ps in self._parts(x, pre))

    def negLogProbability(self, x, pre, average=True):
        s = self.exampleNegLogProbability(x, pre)
        return s.mean() if average else s.sum()

    def generateAtMean(self, pre): return torch.cat([d.generateAtMean(ps) for d, _, ps in self._parts(None, pre)], 1)
    def generateRandom(self, pre): return torch.cat([d.generateRandom(ps) for d, _, ps in self._parts(None, pre)], 1)

    def to_json(self):
        return {"@class": _V + "CompositeReconstructionDistribution", "distributionSizes": self.sizes,
                "reconstructionDistributions": [d.to_json() for d in self.distributions]}


def reconstruction_from_json(d):
    name = d["@class"].rsplit(".", 1)[-1]
    act = Activation.from_json(d["activationFn"]) if d.get("activationFn") is not None else None
    if name == "GaussianReconstructionDistribution":
        return GaussianReconstructionDistribution(act)
    if name == "BernoulliReconstructionDistribution":
        return BernoulliReconstructionDistribution(act)
    if name == "ExponentialReconstructionDistribution":
        return ExponentialReconstructionDistribution(act)
    if name == "LossFunctionWrapper":
        return LossFunctionWrapper(act, LossFunctions.from_json(d["lossFunction"]))
    if name == "CompositeReconstructionDistribution":
        return CompositeReconstructionDistribution(d["distributionSizes"], [reconstruction_from_json(x) for x in d["reconstructionDistributions"]])
    raise ValueError(f"unknown reconstruction distribution {d['@class']}")


# ============================================================================= VAE
class VariationalAutoencoder(FeedForwardLayer):
    """Supervised forward pass = encoder -> mean of q(z|x) (``nOut`` latent values).  ``pretrain_score`` is the
    negative ELBO: KL(q(z|x) || N(0,I)) + E_q[-log p(x|z)] estimated with ``numSamples`` reparameterised samples."""
    JAVA_CLASS = _V + "VariationalAutoencoder"
    DEFAULTS = {"encoderLayerSizes": (100,), "decoderLayerSizes": (100,), "reconstructionDistribution": None,
                "pzxActivationFunction": None, "numSamples": 1}

    def _finalise(self):
        super()._finalise()
        self.encoderLayerSizes = [int(s) for s in (self.encoderLayerSizes if isinstance(self.encoderLayerSizes, (list, tuple)) else [self.encoderLayerSizes])]
        self.decoderLayerSizes = [int(s) for s in (self.decoderLayerSizes if isinstance(self.decoderLayerSizes, (list, tuple)) else [self.decoderLayerSizes])]
        if self.reconstructionDistribution is None:
            self.reconstructionDistribution = GaussianReconstructionDistribution("identity")
        if self.pzxActivationFunction is None:
            self.pzxActivationFunction = Activation.get("identity")
        elif not hasattr(self.pzxActivationFunction, "to_json"):
            self.pzxActivationFunction = Activation.get(self.pzxActivationFunction)

    def _post_json(self):
        if isinstance(self.pzxActivationFunction, dict):
            self.pzxActivationFunction = Activation.from_json(self.pzxActivationFunction)
        self._finalise()

    def param_specs(self):
        s, n_in = [], self.nIn
        for i, n in enumerate(self.encoderLayerSizes):
            s += [ParamSpec(f"e{i}W", (n_in, n), "f", "weight", n_in, n), ParamSpec(f"e{i}b", (1, n), "c", "bias", n_in, n)]
            n_in = n
        for nm in ("pZXMean", "pZXLogStd2"):
            s += [ParamSpec(nm + "W", (n_in, self.nOut), "f", "weight", n_in, self.nOut), ParamSpec(nm + "b", (1, self.nOut), "c", "bias", n_in, self.nOut)]
        n_in = self.nOut
        for i, n in enumerate(self.decoderLayerSizes):
            s += [ParamSpec(f"d{i}W", (n_in, n), "f", "weight", n_in, n), ParamSpec(f"d{i}b", (1, n), "c", "bias", n_in, n)]
            n_in = n
        n_px = self.reconstructionDistribution.distributionInputSize(self.nIn)
        s += [ParamSpec("pXZW", (n_in, n_px), "f", "weight", n_in, n_px), ParamSpec("pXZb", (1, n_px), "c", "bias", n_in, n_px)]
        return s

    def is_pretrain_param(self, name):
        return name.startswith("d") or name.startswith("pXZ") or name.startswith("pZXLogStd2")

    def _encode(self, p, x, training):
        h = x
        for i in range(len(self.encoderLayerSizes)):
            h = self.activation(h @ p[f"e{i}W"] + p[f"e{i}b"], training)
        return h

    def _decode_pre(self, p, z, training):
        h = z
        for i in range(len(self.decoderLayerSizes)):
            h = self.activation(h @ p[f"d{i}W"] + p[f"d{i}b"], training)
        return h @ p["pXZW"] + p["pXZb"]

    def forward(self, p, x, training, mask=None, ctx=None):
        h = self._encode(p, self.apply_dropout(x, training), training)
        return self.pzxActivationFunction(h @ p["pZXMeanW"] + p["pZXMeanb"], training)

    def pretrain_score(self, p, x):
        h = self._encode(p, x, True)
        mean = self.pzxActivationFunction(h @ p["pZXMeanW"] + p["pZXMeanb"], True)
        log_var = self.pzxActivationFunction(h @ p["pZXLogStd2W"] + p["pZXLogStd2b"], True)
        kl = 0.5 * (log_var.exp() + mean ** 2 - 1.0 - log_var).sum(1).mean()
        rec = 0.0
        for _ in range(self.numSamples):
            z = mean + torch.randn_like(mean) * (0.5 * log_var).exp()
            rec = rec + self.reconstructionDistribution.negLogProbability(x, self._decode_pre(p, z, True), True)
        return kl + rec / self.numSamples

    # -- generation / scoring helpers (VariationalAutoencoder.java: reconstructionLogProbability, generateAtMeanGivenZ ...)
    def reconstructionLogProbability(self, p, x, numSamples=5):
        with torch.no_grad():
            h = self._encode(p, x, False)
            mean = self.pzxActivationFunction(h @ p["pZXMeanW"] + p["pZXMeanb"], False)
            log_var = self.pzxActivationFunction(h @ p["pZXLogStd2W"] + p["pZXLogStd2b"], False)
            lps = []
            for _ in range(numSamples):
                z = mean + torch.randn_like(mean) * (0.5 * log_var).exp()
                lps.append(-self.reconstructionDistribution.exampleNegLogProbability(x, self._decode_pre(p, z, False)))
            return torch.logsumexp(torch.stack(lps), 0) - math.log(numSamples)

    def reconstructionProbability(self, p, x, numSamples=5): return self.reconstructionLogProbability(p, x, numSamples).exp()
    def generateAtMeanGivenZ(self, p, z): return self.reconstructionDistribution.generateAtMean(self._decode_pre(p, z, False))
    def generateRandomGivenZ(self, p, z): return self.reconstructionDistribution.generateRandom(self._decode_pre(p, z, False))
    def hasLossFunction(self): return self.reconstructionDistribution.hasLossFunction()

    def reconstructionError(self, p, x):
        if not self.hasLossFunction():
            raise ValueError("reconstructionError needs a LossFunctionWrapper reconstruction distribution; use reconstructionProbability")
        return self.reconstructionDistribution.exampleNegLogProbability(x, self._decode_pre(p, self.forward(p, x, False), False))


# ============================================================================= locally connected
class LocallyConnected2D(BaseLayer):
    """Convolution with untied weights: one [kH*kW*nIn, nOut] filter bank per output position."""
    JAVA_CLASS = _L + "LocallyConnected2D"
    DEFAULTS = {"nIn": 0, "nOut": 0, "kernel": (2, 2), "stride": (1, 1), "padding": (0, 0), "dilation": (1, 1), "convolutionMode": "Same",
                "hasBias": True, "inputSize": None, "format": "NCHW"}

    def _finalise(self):
        super()._finalise()
        for k in ("kernel", "stride", "padding", "dilation"):
            v = getattr(self, k)
            setattr(self, k, tuple(int(x) for x in (v if isinstance(v, (list, tuple)) else (v, v))))

    def setNIn(self, it, override):
        if it.kind == InputType.CNN:
            if not self.nIn or override:
                self.nIn = it.channels
            self.inputSize = (it.height, it.width)

    def _geometry(self):
        h, w = self.inputSize
        same = str(self.convolutionMode).lower().endswith("same")
        if same:
            oh, ow = math.ceil(h / self.stride[0]), math.ceil(w / self.stride[1])
            ph = max((oh - 1) * self.stride[0] + (self.kernel[0] - 1) * self.dilation[0] + 1 - h, 0)
            pw = max((ow - 1) * self.stride[1] + (self.kernel[1] - 1) * self.dilation[1] + 1 - w, 0)
            pad = (pw // 2, pw - pw // 2, ph // 2, ph - ph // 2)
        else:
            oh = (h + 2 * self.padding[0] - self.dilation[0] * (self.kernel[0] - 1) - 1) // self.stride[0] + 1
            ow = (w + 2 * self.padding[1] - self.dilation[1] * (self.kernel[1] - 1) - 1) // self.stride[1] + 1
            pad = (self.padding[1], self.padding[1], self.padding[0], self.padding[0])
        return oh, ow, pad

    def output_type(self, it):
        oh, ow, _ = self._geometry()
        return InputType.convolutional(oh, ow, self.nOut)

    def param_specs(self):
        oh, ow, _ = self._geometry()
        fan = self.kernel[0] * self.kernel[1] * self.nIn
        s = [ParamSpec("W", (oh * ow, fan, self.nOut), "c", "weight", fan, self.nOut)]
        if self.hasBias:
            s.append(ParamSpec("b", (1, self.nOut), "c", "bias", fan, self.nOut))
        return s

    def forward(self, p, x, training, mask=None, ctx=None):
        oh, ow, pad = self._geometry()
        x = F.pad(self.apply_dropout(x, training), pad)
        cols = F.unfold(x, self.kernel, dilation=self.dilation, stride=self.stride)          # [N, nIn*kH*kW, L]
        out = torch.einsum("nfl,lfo->nol", cols, p["W"].to(cols.dtype))
        if self.hasBias:
            out = out + p["b"].reshape(1, -1, 1).to(out.dtype)
        return self.activation(out.reshape(x.shape[0], self.nOut, oh, ow), training)


class LocallyConnected1D(BaseLayer):
    JAVA_CLASS = _L + "LocallyConnected1D"
    DEFAULTS = {"nIn": 0, "nOut": 0, "kernel": 2, "stride": 1, "padding": 0, "dilation": 1, "convolutionMode": "Same", "hasBias": True,
                "inputSize": None}

    def setNIn(self, it, override):
        if it.kind == InputType.RNN:
            if not self.nIn or override:
                self.nIn = it.size
            if it.timeSeriesLength and it.timeSeriesLength > 0:
                self.inputSize = it.timeSeriesLength

    def _geometry(self):
        t = int(self.inputSize)
        if str(self.convolutionMode).lower().endswith("same"):
            ot = math.ceil(t / self.stride)
            pt = max((ot - 1) * self.stride + (self.kernel - 1) * self.dilation + 1 - t, 0)
            return ot, (pt // 2, pt - pt // 2)
        return (t + 2 * self.padding - self.dilation * (self.kernel - 1) - 1) // self.stride + 1, (self.padding, self.padding)

    def output_type(self, it):
        return InputType.recurrent(self.nOut, self._geometry()[0])

    def param_specs(self):
        ot, _ = self._geometry()
        fan = self.kernel * self.nIn
        s = [ParamSpec("W", (ot, fan, self.nOut), "c", "weight", fan, self.nOut)]
        if self.hasBias:
            s.append(ParamSpec("b", (1, self.nOut), "c", "bias", fan, self.nOut))
        return s

    def forward(self, p, x, training, mask=None, ctx=None):
        ot, pad = self._geometry()
        x = F.pad(self.apply_dropout(x, training), pad)                                       # [N, C, T]
        cols = F.unfold(x.unsqueeze(2), (1, self.kernel), dilation=(1, self.dilation), stride=(1, self.stride))
        out = torch.einsum("nfl,lfo->nol", cols, p["W"].to(cols.dtype))
        if self.hasBias:
            out = out + p["b"].reshape(1, -1, 1).to(out.dtype)
        return self.activation(out, training)


# ============================================================================= capsules
def _squash(s, dim=-1, eps=1e-8):
    n2 = (s * s).sum(dim, keepdim=True)
    return s * (n2 / (1.0 + n2)) / torch.sqrt(n2 + eps)


class PrimaryCapsules(BaseLayer):
    """Convolution whose output channels are grouped into ``capsules`` x ``capsuleDimensions`` and squashed;
    output [N, totalCapsules, capsuleDimensions]."""
    JAVA_CLASS = _L + "PrimaryCapsules"
    DEFAULTS = {"kernelSize": (9, 9), "stride": (2, 2), "padding": (0, 0), "dilation": (1, 1), "convolutionMode": "Truncate",
                "useRelu": False, "leak": 0.0, "capsuleDimensions": 8, "channels": 32, "inputChannels": 0, "capsules": 0, "hasBias": True,
                "inputSize": None}

    def _positional(self, *a):
        if a:
            self.capsuleDimensions, self.channels = int(a[0]), int(a[1])

    def setNIn(self, it, override):
        if it.kind == InputType.CNN:
            self.inputChannels = it.channels
            self.inputSize = (it.height, it.width)
            oh, ow = self._out_hw()
            self.capsules = self.channels * oh * ow

    def _tup(self, v): return tuple(int(x) for x in (v if isinstance(v, (list, tuple)) else (v, v)))

    def _out_hw(self):
        k, s, pd, d = (self._tup(getattr(self, n)) for n in ("kernelSize", "stride", "padding", "dilation"))
        h, w = self.inputSize
        if str(self.convolutionMode).lower().endswith("same"):
            return math.ceil(h / s[0]), math.ceil(w / s[1])
        return ((h + 2 * pd[0] - d[0] * (k[0] - 1) - 1) // s[0] + 1, (w + 2 * pd[1] - d[1] * (k[1] - 1) - 1) // s[1] + 1)

    def output_type(self, it): return InputType.recurrent(self.capsuleDimensions, self.capsules, "NWC")

    def param_specs(self):
        k = self._tup(self.kernelSize)
        co = self.capsuleDimensions * self.channels
        fan_in = self.inputChannels * k[0] * k[1]
        s = [ParamSpec("W", (co, self.inputChannels, k[0], k[1]), "c", "weight", fan_in, co * k[0] * k[1])]
        if self.hasBias:
            s.append(ParamSpec("b", (1, co), "c", "bias", fan_in, co))
        return s

    def forward(self, p, x, training, mask=None, ctx=None):
        k, s, pd, d = (self._tup(getattr(self, n)) for n in ("kernelSize", "stride", "padding", "dilation"))
        if str(self.convolutionMode).lower().endswith("same"):
            oh, ow = self._out_hw()
            ph = max((oh - 1) * s[0] + (k[0] - 1) * d[0] + 1 - x.shape[2], 0)
            pw = max((ow - 1) * s[1] + (k[1] - 1) * d[1] + 1 - x.shape[3], 0)
            x, pd = F.pad(x, (pw // 2, pw - pw // 2, ph // 2, ph - ph // 2)), (0, 0)
        y = F.conv2d(x, p["W"].to(x.dtype), p["b"].reshape(-1).to(x.dtype) if self.hasBias else None, s, pd, d)
        if self.useRelu:
            y = F.leaky_relu(y, self.leak) if self.leak else F.relu(y)
        n = y.shape[0]
        caps = y.reshape(n, self.channels, self.capsuleDimensions, -1).permute(0, 1, 3, 2).reshape(n, -1, self.capsuleDimensions)
        return _squash(caps)


class CapsuleLayer(BaseLayer):
    """Dynamic routing between capsules (Sabour et al.): input [N, inputCapsules, inputCapsuleDimensions] ->
    [N, capsules, capsuleDimensions]."""
    JAVA_CLASS = _L + "CapsuleLayer"
    DEFAULTS = {"hasBias": False, "inputCapsules": 0, "inputCapsuleDimensions": 0, "capsules": 0, "capsuleDimensions": 0, "routings": 3}

    def _positional(self, *a):
        if a:
            self.capsules, self.capsuleDimensions = int(a[0]), int(a[1])
            if len(a) > 2:
                self.routings = int(a[2])

    def setNIn(self, it, override):
        if it.kind == InputType.RNN:
            self.inputCapsules, self.inputCapsuleDimensions = int(it.timeSeriesLength), int(it.size)

    def output_type(self, it): return InputType.recurrent(self.capsuleDimensions, self.capsules, "NWC")

    def param_specs(self):
        fan_in = self.inputCapsules * self.inputCapsuleDimensions
        s = [ParamSpec("weight", (1, self.inputCapsules, self.capsules * self.capsuleDimensions, self.inputCapsuleDimensions), "c", "weight",
                       fan_in, self.capsules * self.capsuleDimensions)]
        if self.hasBias:
            s.append(ParamSpec("bias", (1, 1, self.capsules, self.capsuleDimensions), "c", "bias", fan_in, self.capsules))
        return s

    def forward(self, p, x, training, mask=None, ctx=None):
        n = x.shape[0]
        W = p["weight"].to(x.dtype)[0]                                                     # [inCaps, caps*capDim, inDim]
        u_hat = torch.einsum("icd,nid->nic", W, x).reshape(n, self.inputCapsules, self.capsules, self.capsuleDimensions)
        b = torch.zeros(n, self.inputCapsules, self.capsules, 1, dtype=x.dtype, device=x.device)
        v = None
        for r in range(self.routings):
            c = torch.softmax(b, dim=2)
            s = (c * u_hat).sum(1, keepdim=True)                                              # [N,1,caps,capDim]
            if self.hasBias:
                s = s + p["bias"].to(x.dtype)
            v = _squash(s, dim=3)
            if r < self.routings - 1:
                b = b + (u_hat * v).sum(3, keepdim=True)
        return v.squeeze(1)


class CapsuleStrengthLayer(NoParamLayer):
    """L2 norm of every capsule: [N, caps, dims] -> [N, caps]."""
    JAVA_CLASS = _L + "CapsuleStrengthLayer"

    def output_type(self, it): return InputType.feedForward(int(it.timeSeriesLength))
    def forward(self, p, x, training, mask=None, ctx=None): return torch.sqrt((x * x).sum(2) + 1e-12)


# ============================================================================= YOLOv2
class Yolo2OutputLayer(NoParamLayer):
    """YOLOv2 loss (``objdetect/Yolo2OutputLayer.java``).  Input [N, B*(5+C), H, W]; labels [N, 4+C, H, W] with
    (x1, y1, x2, y2) in grid units followed by a one-hot class map.  Per box the network predicts
    (tx, ty, tw, th, conf): centre = sigmoid(txy) + cell, size = prior * exp(twh), confidence = sigmoid(conf), with
    a softmax over classes.  The responsible box in an object cell is the one with the highest IOU."""
    JAVA_CLASS = _L + "objdetect.Yolo2OutputLayer"
    DEFAULTS = {"lambdaCoord": 5.0, "lambdaNoObj": 0.5, "lossPositionScale": None, "lossClassPredictions": None, "boundingBoxes": None}
    IS_OUTPUT = True
    JSON_SKIP = ()

    def _finalise(self):
        super()._finalise()
        if self.boundingBoxes is not None and not isinstance(self.boundingBoxes, torch.Tensor):
            self.boundingBoxes = torch.as_tensor(self.boundingBoxes, dtype=torch.float32).reshape(-1, 2)
        for k in ("lossPositionScale", "lossClassPredictions"):
            v = getattr(self, k)
            if v is None:
                setattr(self, k, LossFunctions.get("L2"))
            elif not isinstance(v, ILossFunction):
                setattr(self, k, LossFunctions.get(v))

    def to_json(self):
        d = super().to_json()
        d["boundingBoxes"] = None if self.boundingBoxes is None else torch.as_tensor(self.boundingBoxes).tolist()
        return d

    def _post_json(self):
        self._finalise()

    def boundingBoxPriors(self, priors):
        self.boundingBoxes = torch.as_tensor(priors, dtype=torch.float32).reshape(-1, 2)
        return self

    def output_type(self, it): return it

    def _decode(self, x):
        nb = self.boundingBoxes.shape[0]
        n, ch, h, w = x.shape
        c = ch // nb - 5
        x5 = x.float().reshape(n, nb, 5 + c, h, w)
        gy, gx = torch.meshgrid(torch.arange(h, device=x.device, dtype=torch.float32), torch.arange(w, device=x.device, dtype=torch.float32), indexing="ij")
        pri = self.boundingBoxes.to(x.device)
        cxy = torch.sigmoid(x5[:, :, 0:2]) + torch.stack([gx, gy])[None, None]
        wh = pri[None, :, :, None, None] * torch.exp(x5[:, :, 2:4])
        conf = torch.sigmoid(x5[:, :, 4])
        cls = torch.softmax(x5[:, :, 5:], dim=2) if c > 0 else x5[:, :, 5:]
        return cxy, wh, conf, cls, x5

    def forward(self, p, x, training, mask=None, ctx=None):
        if ctx is not None:
            ctx["preout"] = x
        cxy, wh, conf, cls, x5 = self._decode(x)
        n, nb = x5.shape[:2]
        return torch.cat([cxy, wh, conf.unsqueeze(2), cls], 2).reshape(n, -1, x.shape[2], x.shape[3]).to(x.dtype)

    def score_from_preout(self, preout, labels, mask=None, average=True, minibatch=None):
        cxy, wh, conf, cls, _ = self._decode(preout)
        labels = labels.float()
        n, nb = cxy.shape[:2]
        tl, br = labels[:, 0:2], labels[:, 2:4]
        obj = ((br - tl).abs().sum(1) > 0).float()                                            # [N,H,W]
        lc, lwh = 0.5 * (tl + br), (br - tl)
        # IOU of every predicted box with the cell's label box
        p_tl, p_br = cxy - 0.5 * wh, cxy + 0.5 * wh
        i_tl = torch.maximum(p_tl, tl[:, None])
        i_br = torch.minimum(p_br, br[:, None])
        inter = (i_br - i_tl).clamp(min=0).prod(2)
        union = wh.prod(2) + lwh.prod(1)[:, None] - inter
        iou = (inter / union.clamp(min=1e-9)) * obj[:, None]
        resp = F.one_hot(iou.argmax(1), nb).permute(0, 3, 1, 2).float() * obj[:, None]         # [N,B,H,W]
        noobj = 1.0 - resp
        pos = ((cxy - lc[:, None]) ** 2).sum(2) + ((wh.clamp(min=1e-9).sqrt() - lwh.clamp(min=1e-9).sqrt()[:, None]) ** 2).sum(2)
        loss = self.lambdaCoord * (resp * pos).sum()
        loss = loss + (resp * (conf - iou.detach()) ** 2).sum() + self.lambdaNoObj * (noobj * conf ** 2).sum()
        if cls.shape[2] > 0:
            lcls = labels[:, 4:]
            loss = loss + (resp[:, :, None] * (cls - lcls[:, None]) ** 2).sum()
        return loss / n if average else loss

    def score_array(self, preout, labels, mask=None):
        return torch.stack([self.score_from_preout(preout[i:i + 1], labels[i:i + 1], None, False) for i in range(preout.shape[0])])

    def getPredictedObjects(self, networkOutput, threshold):
        """Decoded detections above ``threshold``: list of dicts (example, centre, size, confidence, class probabilities)."""
        out = getattr(networkOutput, "t", networkOutput)
        nb = self.boundingBoxes.shape[0]
        n, ch, h, w = out.shape
        o = out.float().reshape(n, nb, ch // nb, h, w)
        res = []
        for idx in (o[:, :, 4] > threshold).nonzero().tolist():
            e, b, y, x = idx
            v = o[e, b, :, y, x]
            res.append({"exampleNumber": e, "centerX": float(v[0]), "centerY": float(v[1]), "width": float(v[2]), "height": float(v[3]),
                        "confidence": float(v[4]), "classPredictions": v[5:].tolist(), "predictedClass": int(v[5:].argmax()) if v.numel() > 5 else -1})
        return res


# ============================================================================= one-class NN
class OCNNOutputLayer(BaseLayer):
    """One-class neural network output (``ocnn/OCNNOutputLayer.java``): score(x) = V . g(x W); objective
    0.5||W||^2 + 0.5||V||^2 + mean(relu(r - score)) / nu - r, with r tracked as the nu-quantile of the scores."""
    JAVA_CLASS = "org.deeplearning4j.nn.conf.ocnn.OCNNOutputLayer"
    DEFAULTS = {"nIn": 0, "nOut": 1, "hiddenSize": 0, "nu": 0.04, "windowSize": 10000, "initialRValue": 0.1, "configureR": True,
                "lossFunction": None}
    IS_OUTPUT = True

    def setNIn(self, it, override):
        if not self.nIn or override:
            self.nIn = it.size if it.kind in (InputType.FF, InputType.RNN) else it.arrayElementsPerExample()

    def output_type(self, it): return InputType.feedForward(1)

    def param_specs(self):
        return [ParamSpec("W", (self.nIn, self.hiddenSize), "f", "weight", self.nIn, self.hiddenSize),
                ParamSpec("V", (self.hiddenSize, 1), "f", "weight", self.hiddenSize, 1),
                ParamSpec("R", (1, 1), "c", "bias", 1, 1, init=float(self.initialRValue))]

    def forward(self, p, x, training, mask=None, ctx=None):
        y = self.activation(x @ p["W"], training) @ p["V"]
        if ctx is not None:
            ctx["preout"] = y
            ctx["ocnn_params"] = p
        return y

    def score_from_preout(self, preout, labels, mask=None, average=True, minibatch=None):
        self._last_scores = preout.detach()
        return preout.sum() * 0.0          # data term added in extra_score, where the parameters are visible

    def extra_score(self, ctx, labels):
        p, y = ctx["ocnn_params"], ctx["preout"]
        if self.configureR:
            # .data: the parameter views of a network share one version counter with the flat buffer
            p["R"].data.fill_(float(torch.quantile(y.detach().float().reshape(-1), self.nu)))
        r = p["R"].reshape(())
        return 0.5 * (p["W"] ** 2).sum() + 0.5 * (p["V"] ** 2).sum() + F.relu(r - y).mean() / self.nu - r

    def score_array(self, preout, labels, mask=None): return preout.reshape(-1)


# ============================================================================= SameDiff-defined layers
class AbstractSameDiffLayer(BaseLayer):
    """Base for layers whose forward pass is written against the SameDiff API.  Subclasses implement
    ``defineParameters(params)`` (calling ``params.addWeightParam / addBiasParam``), ``defineLayer(sd, layerInput,
    paramTable, mask)`` returning the output SDVariable, and ``getOutputType``; optionally ``initializeParameters``."""
    JAVA_CLASS = _L + "samediff.AbstractSameDiffLayer"
    DEFAULTS = {}

    class _Params:
        def __init__(self): self.specs = []
        def addWeightParam(self, name, *shape): self.specs.append(ParamSpec(name, tuple(int(s) for s in shape), "c", "weight", shape[0], shape[-1]))
        def addBiasParam(self, name, *shape): self.specs.append(ParamSpec(name, tuple(int(s) for s in shape), "c", "bias", 1, shape[-1]))

    def defineParameters(self, params): pass
    def defineLayer(self, sd, layerInput, paramTable, mask=None): raise NotImplementedError
    def getOutputType(self, layerIndex, inputType): return inputType
    def output_type(self, it): return self.getOutputType(-1, it)

    def param_specs(self):
        pr = self._Params()
        self.defineParameters(pr)
        return pr.specs

    def _graph(self, p, x):
        from ...nd.dtype import DataType
        from ...samediff.core import SameDiff
        key = (tuple(x.shape[1:]), x.dtype)
        cache = self.__dict__.setdefault("_sd_cache", {})
        if key not in cache:
            sd = SameDiff.create()
            inp = sd.placeHolder("input", DataType.from_torch(x.dtype), -1, *x.shape[1:])
            table = {k: sd.placeHolder(k, DataType.from_torch(v.dtype), *v.shape) for k, v in p.items()}
            out = self.defineLayer(sd, inp, table, None)
            cache[key] = (sd, out.name)
        return cache[key]

    def forward(self, p, x, training, mask=None, ctx=None):
        from ...samediff.session import InferenceSession
        sd, out = self._graph(p, x)
        sd.device = x.device
        vals = InferenceSession(sd).run({"input": x, **p}, [out], None, training)
        return vals[out]

    def __deepcopy__(self, memo):
        import copy
        c = self.__class__.__new__(self.__class__)
        memo[id(self)] = c
        for k, v in self.__dict__.items():
            if k != "_sd_cache":
                setattr(c, k, copy.deepcopy(v, memo))
        return c


class SameDiffLayer(AbstractSameDiffLayer):
    JAVA_CLASS = _L + "samediff.SameDiffLayer"


class SameDiffLambdaLayer(AbstractSameDiffLayer):
    """Parameter-free SameDiff layer: implement ``defineLayer(sd, layerInput)``."""
    JAVA_CLASS = _L + "samediff.SameDiffLambdaLayer"
    HAS_PARAMS = False

    def param_specs(self): return []

    def _graph(self, p, x):
        from ...nd.dtype import DataType
        from ...samediff.core import SameDiff
        key = (tuple(x.shape[1:]), x.dtype)
        cache = self.__dict__.setdefault("_sd_cache", {})
        if key not in cache:
            sd = SameDiff.create()
            inp = sd.placeHolder("input", DataType.from_torch(x.dtype), -1, *x.shape[1:])
            cache[key] = (sd, self.defineLayer(sd, inp).name)
        return cache[key]


class SameDiffOutputLayer(AbstractSameDiffLayer):
    """SameDiff-defined output layer: ``defineLayer(sd, layerInput, labels, paramTable)`` returns the scalar loss
    variable; ``activationsVertexName()`` names the variable holding the predictions."""
    JAVA_CLASS = _L + "samediff.SameDiffOutputLayer"
    IS_OUTPUT = True

    def activationsVertexName(self): raise NotImplementedError
    def labelsRequired(self): return True

    def _graph_out(self, p, x, labels):
        from ...nd.dtype import DataType
        from ...samediff.core import SameDiff
        key = (tuple(x.shape[1:]), x.dtype, None if labels is None else tuple(labels.shape[1:]))
        cache = self.__dict__.setdefault("_sd_cache", {})
        if key not in cache:
            sd = SameDiff.create()
            inp = sd.placeHolder("input", DataType.from_torch(x.dtype), -1, *x.shape[1:])
            lab = sd.placeHolder("labels", DataType.FLOAT, -1, *(labels.shape[1:] if labels is not None else ()))
            table = {k: sd.placeHolder(k, DataType.from_torch(v.dtype), *v.shape) for k, v in p.items()}
            loss = self.defineLayer(sd, inp, lab, table)
            cache[key] = (sd, loss.name)
        return cache[key]

    def forward(self, p, x, training, mask=None, ctx=None):
        from ...samediff.session import InferenceSession
        if ctx is not None:
            ctx["preout"] = x
        self.__dict__["_score_params"] = p
        dummy = torch.zeros((x.shape[0],) + tuple(self._label_shape or ()), device=x.device) if getattr(self, "_label_shape", None) is not None else None
        sd, _ = self._graph_out(p, x, dummy if dummy is not None else torch.zeros(x.shape[0], 1, device=x.device))
        sd.device = x.device
        name = self.activationsVertexName()
        ph = {"input": x, **p}
        return InferenceSession(sd).run(ph, [name], None, training)[name]

    def score_from_preout(self, preout, labels, mask=None, average=True, minibatch=None):
        from ...samediff.session import InferenceSession
        p = self._score_params
        self._label_shape = tuple(labels.shape[1:])
        sd, loss = self._graph_out(p, preout, labels)
        sd.device = preout.device
        return InferenceSession(sd).run({"input": preout, "labels": labels, **p}, [loss], None, True)[loss].sum()

    def extra_score(self, ctx, labels):
        return 0.0


__all__ = [n for n, v in list(globals().items()) if isinstance(v, type) and (issubclass(v, Layer) or issubclass(v, ReconstructionDistribution))]
