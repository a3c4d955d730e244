"""Loss ops (``headers/loss.h``) with the TF-style ``reductionMode`` of the native implementations
(``libnd4j/include/ops/declarable/generic/loss/*.cpp``): 0 = none, 1 = sum, 2 = mean by total
weight, 3 = mean by the number of non-zero weights.  ``*_grad`` ops return (dPredictions, dWeights,
dLabels) like the native ones."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import nnops
from .registry import op

NONE, SUM, MEAN_BY_WEIGHT, MEAN_BY_NONZERO_WEIGHT_COUNT = 0, 1, 2, 3


def _mode(m):
    if isinstance(m, str):
        return {"NONE": 0, "SUM": 1, "MEAN_BY_WEIGHT": 2, "MEAN_BY_NONZERO_WEIGHT_COUNT": 3}[m.upper()]
    return int(m)


def _reduce(per, w, mode):
    mode = _mode(mode)
    if w is None:
        w = torch.ones((), dtype=per.dtype, device=per.device)
    w = w.to(per.dtype)
    e = per * w
    if mode == NONE:
        return e
    s = e.sum()
    if mode == SUM:
        return s
    wb = w.expand_as(per) if w.dim() else w
    if mode == MEAN_BY_WEIGHT:
        tot = wb.sum() if w.dim() else w * per.numel()
        return s / tot
    cnt = (wb != 0).sum().clamp_min(1) if w.dim() else torch.tensor(per.numel() if float(w) != 0 else 1, device=per.device)
    return s / cnt


def _grad3(fn):
    def run(pred, weights, labels, **kw):
        p = pred.detach().requires_grad_(True)
        w = weights.detach().float().requires_grad_(True) if weights is not None else None
        l = labels.detach().float().requires_grad_(True) if labels.dtype.is_floating_point else labels
        with torch.enable_grad():
            y = fn(p, w, l, **kw)
            y = y.sum() if y.dim() else y
        ins = [t for t in (p, w, l) if t is not None and t.requires_grad]
        gs = list(torch.autograd.grad(y, ins, allow_unused=True))
        out = []
        for t in (p, w, l):
            if t is not None and t.requires_grad:
                g = gs.pop(0)
                out.append(g if g is not None else torch.zeros_like(t))
            else:
                out.append(torch.zeros_like(t, dtype=torch.float32) if t is not None else None)
        return tuple(out)
    return run


def _loss(name, per_fn):
    def fwd(pred, weights, labels, reductionMode=MEAN_BY_NONZERO_WEIGHT_COUNT, **kw):
        return _reduce(per_fn(pred, labels, **kw), weights, reductionMode)
    op(name)(fwd)
    op(name + "_grad", n_out=3)(_grad3(fwd))
    return fwd


_loss("absolute_difference_loss", lambda p, l, **kw: (p - l).abs())
_loss("mean_sqerr_loss", lambda p, l, **kw: (p - l) ** 2)
_loss("hinge_loss", lambda p, l, **kw: F.relu(1 - (2 * l - 1) * p))
_loss("huber_loss", lambda p, l, delta=1.0, **kw: torch.where((p - l).abs() <= delta, 0.5 * (p - l) ** 2, delta * (p - l).abs() - 0.5 * delta * delta))
_loss("log_loss", lambda p, l, epsilon=1e-7, **kw: -(l * torch.log(p + epsilon) + (1 - l) * torch.log(1 - p + epsilon)))
_loss("log_poisson_loss", lambda p, l, full=False, **kw: torch.exp(p) - l * p + ((l * torch.log(l.clamp_min(1e-30)) - l + 0.5 * torch.log(2 * torch.pi * l.clamp_min(1e-30))) * (l > 1) if full else 0))
_loss("sigm_cross_entropy_loss", lambda p, l, labelsSmoothing=0.0, **kw: F.binary_cross_entropy_with_logits(p, l * (1 - labelsSmoothing) + 0.5 * labelsSmoothing, reduction="none"))
_loss("cosine_distance_loss", lambda p, l, dimension=-1, **kw: 1 - (p * l).sum(int(dimension), keepdim=True))


def _mpwse(p, l, **kw):
    d = (p - l).reshape(p.shape[0], -1)
    n = d.shape[1]
    s1 = (d * d).sum(1)
    s2 = d.sum(1) ** 2
    return (2.0 * (n * s1 - s2) / max(n * (n - 1), 1)).reshape(-1, 1)


_loss("mean_pairwssqerr_loss", _mpwse)

op("l2_loss")(lambda x, **kw: 0.5 * (x * x).sum())


@op("softmax_cross_entropy_loss")
def softmax_cross_entropy_loss(logits, weights, labels, reductionMode=MEAN_BY_NONZERO_WEIGHT_COUNT, labelsSmoothing=0.0, **kw):
    if labelsSmoothing:
        labels = labels * (1 - labelsSmoothing) + labelsSmoothing / labels.shape[-1]
    if logits.dim() == 2:
        per = nnops.softmax_xent(logits, labels, sparse=False)
    else:
        per = -(labels.to(torch.float32) * F.log_softmax(logits.float(), -1)).sum(-1)
    w = weights
    if w is not None and w.dim() == per.dim() + 1:
        w = w.squeeze(-1)
    return _reduce(per, w, reductionMode)


op("softmax_cross_entropy_loss_grad", n_out=3)(_grad3(softmax_cross_entropy_loss))


@op("softmax_cross_entropy_loss_with_logits")
def softmax_cross_entropy_loss_with_logits(logits, labels, classesDim=-1, **kw):
    d = int(classesDim) % logits.dim()
    if d == logits.dim() - 1 and logits.dim() == 2:
        return nnops.softmax_xent(logits, labels, sparse=False)
    return -(labels.to(torch.float32) * F.log_softmax(logits.float(), d)).sum(d)


@op("softmax_cross_entropy_loss_with_logits_grad", n_out=2)
def softmax_cross_entropy_loss_with_logits_grad(logits, labels, classesDim=-1, **kw):
    d = int(classesDim) % logits.dim()
    p = torch.softmax(logits.float(), d)
    return (p * labels.sum(d, keepdim=True) - labels).to(logits.dtype), -F.log_softmax(logits.float(), d).to(logits.dtype)


@op("sparse_softmax_cross_entropy_loss_with_logits")
def sparse_softmax_cross_entropy_loss_with_logits(labels, logits, **kw):
    """Note the native argument order: (labels, logits)."""
    if labels.dtype.is_floating_point and labels.dim() == logits.dim():   # tolerate (logits, labels)
        labels, logits = logits, labels
    if logits.dim() == 2:
        return nnops.softmax_xent(logits, labels.reshape(-1), sparse=True)
    lp = F.log_softmax(logits.float(), -1)
    return -lp.gather(-1, labels.long().unsqueeze(-1)).squeeze(-1)


@op("sparse_softmax_cross_entropy_loss_with_logits_grad")
def sparse_softmax_cross_entropy_loss_with_logits_grad(labels, logits, **kw):
    p = torch.softmax(logits.float(), -1)
    return (p - F.one_hot(labels.long(), logits.shape[-1]).to(p.dtype)).to(logits.dtype)


@op("weighted_cross_entropy_with_logits")
def weighted_cross_entropy_with_logits(targets, logits, weights, **kw):
    lw = 1 + (weights - 1) * targets
    return (1 - targets) * logits + lw * (torch.log1p(torch.exp(-logits.abs())) + F.relu(-logits))


@op("ctc_loss")
def ctc_loss(targetLabels, logitInput, targetLabelLengths, logitInputLengths, blankIndex=0, **kw):
    """logitInput [B, T, C] (batch-major, as the native op); returns the per-example loss [B]."""
    lp = F.log_softmax(logitInput if logitInput.dtype == torch.float64 else logitInput.float(), -1).permute(1, 0, 2)
    return F.ctc_loss(lp, targetLabels.long(), logitInputLengths.long(), targetLabelLengths.long(), blank=int(blankIndex),
                      reduction="none", zero_infinity=False)


@op("ctc_loss_grad")
def ctc_loss_grad(targetLabels, logitInput, targetLabelLengths, logitInputLengths, blankIndex=0, **kw):
    x = logitInput.detach().float().requires_grad_(True)
    with torch.enable_grad():
        l = ctc_loss(targetLabels, x, targetLabelLengths, logitInputLengths, blankIndex).sum()
    return torch.autograd.grad(l, x)[0].to(logitInput.dtype)


@op("ctc_beam", n_out=3, differentiable=False)
def ctc_beam(logits, seqLengths, blankIndex=0, beamWidth=25, nbestSize=1, normalizeLogits=True, **kw):
    """Prefix beam search over [B, T, C] log-probabilities; returns (sequences [B, nbest, T],
    log-probabilities [B, nbest], lengths [B, nbest]) (``helpers/impl/ctcBeam.cpp``)."""
    import math
    lp = F.log_softmax(logits.float(), -1) if normalizeLogits else logits.float()
    B, T, C = lp.shape
    blank, W, nb = int(blankIndex), int(beamWidth), int(nbestSize)
    seqs = torch.full((B, nb, T), -1, dtype=torch.int64)
    probs = torch.full((B, nb), float("-inf"))
    lens = torch.zeros((B, nb), dtype=torch.int64)
    lpc = lp.cpu()

    def lse(a, b):
        if a == float("-inf"):
            return b
        if b == float("-inf"):
            return a
        m = max(a, b)
        return m + math.log(math.exp(a - m) + math.exp(b - m))
    for b in range(B):
        beams = {(): (0.0, float("-inf"))}     # prefix -> (log p ending in blank, log p ending in non-blank)
        for t in range(int(seqLengths[b])):
            row = lpc[b, t].tolist()
            nxt = {}
            for pre, (pb, pnb) in beams.items():
                tot = lse(pb, pnb)
                e = nxt.get(pre, (float("-inf"), float("-inf")))
                nxt[pre] = (lse(e[0], tot + row[blank]), e[1])
                for c in range(C):
                    if c == blank:
                        continue
                    npre = pre + (c,)
                    e = nxt.get(npre, (float("-inf"), float("-inf")))
                    if pre and pre[-1] == c:
                        nxt[npre] = (e[0], lse(e[1], pb + row[c]))
                        e2 = nxt.get(pre, (float("-inf"), float("-inf")))
                        nxt[pre] = (e2[0], lse(e2[1], pnb + row[c]))
                    else:
                        nxt[npre] = (e[0], lse(e[1], tot + row[c]))
            beams = dict(sorted(nxt.items(), key=lambda kv: -lse(*kv[1]))[:W])
        best = sorted(beams.items(), key=lambda kv: -lse(*kv[1]))[:nb]
        for i, (pre, pr) in enumerate(best):
            seqs[b, i, :len(pre)] = torch.tensor(pre, dtype=torch.int64) if pre else seqs[b, i, :0]
            probs[b, i] = lse(*pr)
            lens[b, i] = len(pre)
    return seqs.to(logits.device), probs.to(logits.device), lens.to(logits.device)
