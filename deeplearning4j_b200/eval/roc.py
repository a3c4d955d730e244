"""ROC / precision-recall evaluation: ``ROC``, ``ROCBinary``, ``ROCMultiClass`` and their curves.

Parity: ``org/nd4j/evaluation/classification/ROC.java`` — ``thresholdSteps == 0`` is the exact mode
(all predictions kept and sorted; AUC by trapezoids over every distinct threshold), ``> 0`` the
thresholded mode (counts at ``steps + 1`` evenly spaced thresholds, mergeable without storing
predictions).  ``ROCBinary`` evaluates each output column independently; ``ROCMultiClass`` is
one-vs-all per class.  The exact mode sorts on the device the predictions live on.
"""
from __future__ import annotations

import torch

from .classification import _t, flatten_time_series


class RocCurve:
    def __init__(self, threshold, fpr, tpr):
        self.threshold, self.fpr, self.tpr = threshold, fpr, tpr

    def getX(self): return self.fpr
    def getY(self): return self.tpr
    def numPoints(self): return len(self.fpr)

    def calculateAUC(self):
        x, y = torch.tensor(self.fpr, dtype=torch.float64), torch.tensor(self.tpr, dtype=torch.float64)
        o = torch.argsort(x, stable=True)
        return float(torch.trapz(y[o], x[o]))


class PrecisionRecallCurve:
    def __init__(self, threshold, precision, recall):
        self.threshold, self.precision, self.recall = threshold, precision, recall

    def getX(self): return self.recall
    def getY(self): return self.precision
    def numPoints(self): return len(self.recall)

    def calculateAUPRC(self):
        x, y = torch.tensor(self.recall, dtype=torch.float64), torch.tensor(self.precision, dtype=torch.float64)
        o = torch.argsort(x, stable=True)
        return float(torch.trapz(y[o], x[o]))

    def getPointAtThreshold(self, thr):
        i = min(range(len(self.threshold)), key=lambda k: abs(self.threshold[k] - thr))
        return {"threshold": self.threshold[i], "precision": self.precision[i], "recall": self.recall[i]}


class ROC:
    def __init__(self, thresholdSteps=0, rocRemoveRedundantPts=True, exactAllocBlockSize=2048):
        self.thresholdSteps = thresholdSteps
        self.isExact = thresholdSteps == 0
        self.rocRemoveRedundantPts = rocRemoveRedundantPts
        self.reset()

    def reset(self):
        self._probs, self._labels = [], []
        self.countActualPositive = self.countActualNegative = 0
        if not self.isExact:
            self._tp = torch.zeros(self.thresholdSteps + 1, dtype=torch.int64)
            self._fp = torch.zeros(self.thresholdSteps + 1, dtype=torch.int64)
        self._cache = None

    def eval(self, labels, predictions, mask=None, recordMetaData=None):
        labels, preds, mask = flatten_time_series(labels, predictions, mask)
        if preds.dim() == 2 and preds.shape[1] == 2:         # softmax over (negative, positive)
            p, l = preds[:, 1], labels[:, 1]
        else:
            p, l = preds.reshape(-1), labels.reshape(-1)
            if mask is not None:
                keep = mask.reshape(-1) > 0
                p, l = p[keep], l[keep]
        self.evalVector(l, p)

    def evalVector(self, l, p):
        l, p = _t(l), _t(p)
        pos = l > 0.5
        self.countActualPositive += int(pos.sum())
        self.countActualNegative += int((~pos).sum())
        self._cache = None
        if self.isExact:
            self._probs.append(p.detach().double())
            self._labels.append(pos)
        else:
            thr = torch.linspace(0, 1, self.thresholdSteps + 1, device=p.device, dtype=torch.float64)
            pred_pos = p.double()[None, :] >= thr[:, None]
            self._tp += (pred_pos & pos[None, :]).sum(1).cpu()
            self._fp += (pred_pos & ~pos[None, :]).sum(1).cpu()

    def merge(self, o):
        self.countActualPositive += o.countActualPositive
        self.countActualNegative += o.countActualNegative
        self._cache = None
        if self.isExact:
            self._probs += o._probs
            self._labels += o._labels
        else:
            self._tp += o._tp
            self._fp += o._fp
        return self

    def getCountActualPositive(self): return self.countActualPositive
    def getCountActualNegative(self): return self.countActualNegative

    def _points(self):
        """(threshold, tp, fp) tensors from the highest threshold (nothing predicted positive) downwards."""
        if self._cache is not None:
            return self._cache
        if self.isExact:
            if not self._probs:
                z = torch.zeros(1, dtype=torch.float64)
                return z + 1, z, z
            p = torch.cat(self._probs)
            l = torch.cat([x.to(p.device) for x in self._labels])
            order = torch.argsort(p, descending=True, stable=True)
            p, l = p[order], l[order]
            tp = torch.cumsum(l.double(), 0)
            fp = torch.cumsum((~l).double(), 0)
            last = torch.ones_like(p, dtype=torch.bool)
            last[:-1] = p[1:] != p[:-1]                          # one point per distinct threshold
            thr = torch.cat([torch.ones(1, dtype=torch.float64, device=p.device), p[last]]).cpu()
            tp = torch.cat([torch.zeros(1, dtype=torch.float64, device=p.device), tp[last]]).cpu()
            fp = torch.cat([torch.zeros(1, dtype=torch.float64, device=p.device), fp[last]]).cpu()
            if float(thr[-1]) > 0.0:
                thr = torch.cat([thr, torch.zeros(1, dtype=torch.float64)])
                tp = torch.cat([tp, tp[-1:]])
                fp = torch.cat([fp, fp[-1:]])
        else:
            thr = torch.linspace(0, 1, self.thresholdSteps + 1, dtype=torch.float64).flip(0)
            tp, fp = self._tp.double().flip(0), self._fp.double().flip(0)
        self._cache = (thr, tp, fp)
        return self._cache

    def getRocCurve(self):
        thr, tp, fp = self._points()
        tpr = tp / max(self.countActualPositive, 1)
        fpr = fp / max(self.countActualNegative, 1)
        if self.isExact and self.rocRemoveRedundantPts and len(thr) > 2:
            keep = torch.ones(len(thr), dtype=torch.bool)
            same_x = (fpr[1:-1] == fpr[:-2]) & (fpr[1:-1] == fpr[2:])
            same_y = (tpr[1:-1] == tpr[:-2]) & (tpr[1:-1] == tpr[2:])
            keep[1:-1] = ~(same_x | same_y)
            thr, fpr, tpr = thr[keep], fpr[keep], tpr[keep]
        return RocCurve(thr.tolist(), fpr.tolist(), tpr.tolist())

    def getPrecisionRecallCurve(self):
        thr, tp, fp = self._points()
        den = tp + fp
        prec = torch.where(den > 0, tp / den.clamp(min=1), torch.ones_like(tp))
        rec = tp / max(self.countActualPositive, 1)
        return PrecisionRecallCurve(thr.tolist(), prec.tolist(), rec.tolist())

    def calculateAUC(self):
        thr, tp, fp = self._points()
        tpr = tp / max(self.countActualPositive, 1)
        fpr = fp / max(self.countActualNegative, 1)
        return float(torch.trapz(tpr, fpr))

    def calculateAUCPR(self):
        thr, tp, fp = self._points()
        den = tp + fp
        prec = torch.where(den > 0, tp / den.clamp(min=1), torch.ones_like(tp))
        rec = tp / max(self.countActualPositive, 1)
        return float(torch.trapz(prec, rec))

    def scoreForMetric(self, metric):
        return {"AUROC": self.calculateAUC, "AUPRC": self.calculateAUCPR}[str(metric).upper()]()

    def stats(self):
        return f"AUC (Area under ROC Curve):                {self.calculateAUC():.6f}\n" \
               f"AUPRC (Area under Precision/Recall Curve): {self.calculateAUCPR():.6f}" + \
               ("" if self.isExact else f"\n[Note: Thresholded AUC/AUPRC calculation used with {self.thresholdSteps} steps; accuracy may reduced compared to exact mode]")

    def newInstance(self):
        return ROC(self.thresholdSteps, self.rocRemoveRedundantPts)


class _MultiROC:
    def __init__(self, thresholdSteps=0, rocRemoveRedundantPts=True):
        self.thresholdSteps, self.rocRemoveRedundantPts = thresholdSteps, rocRemoveRedundantPts
        self.underlying = None
        self.labels = None

    def reset(self):
        self.underlying = None

    def _ensure(self, n):
        if self.underlying is None:
            self.underlying = [ROC(self.thresholdSteps, self.rocRemoveRedundantPts) for _ in range(n)]

    def merge(self, o):
        if o.underlying is None:
            return self
        self._ensure(len(o.underlying))
        for a, b in zip(self.underlying, o.underlying):
            a.merge(b)
        return self

    def setLabelNames(self, names): self.labels = list(names)
    def getNumClasses(self): return 0 if self.underlying is None else len(self.underlying)
    numLabels = getNumClasses
    def calculateAUC(self, i): return self.underlying[i].calculateAUC()
    def calculateAUCPR(self, i): return self.underlying[i].calculateAUCPR()
    def getRocCurve(self, i): return self.underlying[i].getRocCurve()
    def getPrecisionRecallCurve(self, i): return self.underlying[i].getPrecisionRecallCurve()
    def getCountActualPositive(self, i): return self.underlying[i].countActualPositive
    def getCountActualNegative(self, i): return self.underlying[i].countActualNegative
    def calculateAverageAUC(self): return sum(r.calculateAUC() for r in self.underlying) / len(self.underlying)
    def calculateAverageAUCPR(self): return sum(r.calculateAUCPR() for r in self.underlying) / len(self.underlying)
    calculateAverageAuc = calculateAverageAUC

    def scoreForMetric(self, metric, i=None):
        if i is None:
            return {"AUROC": self.calculateAverageAUC, "AUPRC": self.calculateAverageAUCPR}[str(metric).upper()]()
        return self.underlying[i].scoreForMetric(metric)

    def stats(self):
        rows = [f"{'Label':<12}{'AUC':>10}{'AUPRC':>10}{'# Pos':>10}{'# Neg':>10}"]
        for i, r in enumerate(self.underlying or []):
            nm = self.labels[i] if self.labels else str(i)
            rows.append(f"{nm:<12}{r.calculateAUC():>10.4f}{r.calculateAUCPR():>10.4f}{r.countActualPositive:>10}{r.countActualNegative:>10}")
        if self.underlying:
            rows.append(f"Average AUC: {self.calculateAverageAUC():.4f}")
        return "\n".join(rows)


class ROCBinary(_MultiROC):
    """Independent binary outputs: column ``i`` of the predictions is scored against column ``i`` of the labels."""

    def eval(self, labels, predictions, mask=None, recordMetaData=None):
        labels, preds, mask = flatten_time_series(labels, predictions, mask)
        self._ensure(preds.shape[1])
        for i, r in enumerate(self.underlying):
            l, p = labels[:, i], preds[:, i]
            if mask is not None:
                m = mask[:, i] if mask.dim() == 2 and mask.shape[1] == preds.shape[1] else mask.reshape(-1)
                l, p = l[m > 0], p[m > 0]
            r.evalVector(l, p)


class ROCMultiClass(_MultiROC):
    """One-vs-all ROC per class of a softmax output."""

    def eval(self, labels, predictions, mask=None, recordMetaData=None):
        labels, preds, mask = flatten_time_series(labels, predictions, mask)
        self._ensure(preds.shape[1])
        if labels.dim() == 1 or labels.shape[1] != preds.shape[1]:
            labels = torch.nn.functional.one_hot(labels.reshape(-1).long(), preds.shape[1])
        for i, r in enumerate(self.underlying):
            r.evalVector(labels[:, i], preds[:, i])
