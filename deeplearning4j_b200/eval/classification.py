"""Classification metrics: ``Evaluation``, ``EvaluationBinary``, ``EvaluationCalibration``.

Parity: ``org/nd4j/evaluation/classification/Evaluation.java`` (confusion matrix, macro/micro
averaging, binary positive-class reporting, top-N), ``EvaluationBinary.java`` (independent
sigmoid outputs, per-output counts and decision thresholds), ``EvaluationCalibration.java``
(reliability diagram bins, residual and probability histograms).  All accumulation happens on the
device of the predictions with a single ``bincount`` per batch; only the small count tensors
travel to the host.
"""
from __future__ import annotations

import json
import math

import torch

from ..nd.ndarray import INDArray


def _t(x):
    if x is None:
        return None
    if isinstance(x, INDArray):
        return x.t
    return x if isinstance(x, torch.Tensor) else torch.as_tensor(x)


def flatten_time_series(labels, preds, mask=None):
    """[N,C,T] (NCW) -> [N*T, C], dropping masked steps; [N,C] passes through (per-example mask applied)."""
    labels, preds, mask = _t(labels), _t(preds), _t(mask)
    if preds.dim() == 3:
        n, c, t = preds.shape
        preds = preds.permute(0, 2, 1).reshape(n * t, c)
        labels = labels.permute(0, 2, 1).reshape(n * t, -1)
        if mask is not None:
            if mask.dim() == 3:                       # per-output mask [N,C,T]
                return labels, preds, mask.permute(0, 2, 1).reshape(n * t, -1)
            keep = mask.reshape(n * t) > 0
            return labels[keep], preds[keep], None
        return labels, preds, None
    if preds.dim() > 3:                               # CNN segmentation style [N,C,H,W,...] -> [N*H*W, C]
        c = preds.shape[1]
        preds = preds.movedim(1, -1).reshape(-1, c)
        labels = labels.movedim(1, -1).reshape(-1, labels.shape[1])
        return labels, preds, None
    if mask is not None and mask.dim() <= 2 and mask.numel() == preds.shape[0]:
        keep = mask.reshape(-1) > 0
        return labels[keep], preds[keep], None
    return labels, preds, mask


class EvaluationAveraging:
    Macro = "Macro"
    Micro = "Micro"


class ConfusionMatrix:
    def __init__(self, n):
        self.m = torch.zeros(n, n, dtype=torch.int64)

    def getCount(self, actual, predicted):
        return int(self.m[actual, predicted])

    def getActualTotal(self, c):
        return int(self.m[c].sum())

    def getPredictedTotal(self, c):
        return int(self.m[:, c].sum())

    def toCSV(self):
        return "\n".join(",".join(str(int(v)) for v in row) for row in self.m)


class Evaluation:
    def __init__(self, numClasses=None, labels=None, topN=1, binaryPositiveClass=1, binaryDecisionThreshold=None,
                 costArray=None):
        if isinstance(numClasses, (list, tuple)):
            labels, numClasses = list(numClasses), len(numClasses)
        self.labelsList = list(labels) if labels is not None else None
        self.numClasses = numClasses if numClasses is not None else (len(labels) if labels else None)
        self.topN = topN
        self.binaryPositiveClass = binaryPositiveClass
        self.binaryDecisionThreshold = binaryDecisionThreshold
        self.costArray = _t(costArray)
        self.confusion_ = None
        self.topNCorrectCount = 0
        self.topNTotalCount = 0
        self.numRowCounter = 0

    # ------------------------------------------------------------------ accumulation
    def _ensure(self, c):
        if self.numClasses is None:
            self.numClasses = c
        if self.confusion_ is None:
            self.confusion_ = ConfusionMatrix(self.numClasses)

    def reset(self):
        self.confusion_ = None
        self.topNCorrectCount = self.topNTotalCount = self.numRowCounter = 0

    def eval(self, labels, predictions, mask=None, recordMetaData=None):
        labels, preds, mask = flatten_time_series(labels, predictions, mask)
        if preds.numel() == 0:
            return
        if preds.dim() == 1:
            preds, labels = preds[:, None], labels.reshape(-1, 1)
        c = preds.shape[1]
        if c == 1:                                     # single sigmoid output -> two classes
            thr = 0.5 if self.binaryDecisionThreshold is None else self.binaryDecisionThreshold
            actual = (labels.reshape(-1) > 0.5).long()
            guess = (preds.reshape(-1).float() > thr).long()
            c = 2
        else:
            actual = labels.argmax(1) if labels.dim() == 2 and labels.shape[1] == c else labels.reshape(-1).long()
            p = preds.float()
            if self.binaryDecisionThreshold is not None and c == 2:
                guess = (p[:, 1] > self.binaryDecisionThreshold).long()
            elif self.costArray is not None:
                guess = (p * self.costArray.to(p.device)).argmax(1)
            else:
                guess = p.argmax(1)
            if self.topN > 1:
                top = p.topk(min(self.topN, c), dim=1).indices
                self.topNCorrectCount += int((top == actual[:, None]).any(1).sum())
                self.topNTotalCount += actual.numel()
        self._ensure(c)
        n = self.numClasses
        counts = torch.bincount(actual * n + guess, minlength=n * n).reshape(n, n).cpu()
        self.confusion_.m += counts
        self.numRowCounter += actual.numel()
        if self.topN <= 1:
            self.topNCorrectCount += int(counts.diag().sum())
            self.topNTotalCount += actual.numel()

    def evalTimeSeries(self, labels, predictions, mask=None):
        self.eval(labels, predictions, mask)

    def merge(self, other):
        if other.confusion_ is None:
            return self
        self._ensure(other.numClasses)
        self.confusion_.m += other.confusion_.m
        self.topNCorrectCount += other.topNCorrectCount
        self.topNTotalCount += other.topNTotalCount
        self.numRowCounter += other.numRowCounter
        return self

    # ------------------------------------------------------------------ counts
    def getConfusionMatrix(self):
        return self.confusion_

    def confusionMatrix(self):
        return self.confusion_.m.clone()

    def _m(self):
        return self.confusion_.m if self.confusion_ is not None else torch.zeros(0, 0, dtype=torch.int64)

    def truePositives(self, c=None):
        d = self._m().diag()
        return int(d[c]) if c is not None else {i: int(v) for i, v in enumerate(d)}

    def falsePositives(self, c=None):
        v = self._m().sum(0) - self._m().diag()
        return int(v[c]) if c is not None else {i: int(x) for i, x in enumerate(v)}

    def falseNegatives(self, c=None):
        v = self._m().sum(1) - self._m().diag()
        return int(v[c]) if c is not None else {i: int(x) for i, x in enumerate(v)}

    def trueNegatives(self, c=None):
        m = self._m()
        v = m.sum() - m.sum(0) - m.sum(1) + m.diag()
        return int(v[c]) if c is not None else {i: int(x) for i, x in enumerate(v)}

    def classCount(self, c):
        return int(self._m()[c].sum())

    def getNumRowCounter(self):
        return self.numRowCounter

    # ------------------------------------------------------------------ metrics
    def accuracy(self):
        m = self._m()
        tot = int(m.sum())
        return float(m.diag().sum()) / tot if tot else 0.0

    def topNAccuracy(self):
        return self.topNCorrectCount / self.topNTotalCount if self.topNTotalCount else 0.0

    @staticmethod
    def _ratio(num, den, edge=0.0):
        return num / den if den else edge

    def _is_binary(self):
        return self.numClasses == 2 and self.binaryPositiveClass is not None

    def _averaged(self, per_class, valid, averaging, micro):
        if self._is_binary():
            return per_class(self.binaryPositiveClass)
        if averaging == EvaluationAveraging.Micro:
            return micro()
        vals = [per_class(i) for i in range(self.numClasses) if valid(i)]
        return sum(vals) / len(vals) if vals else 0.0

    def precision(self, c=None, edgeCase=0.0, averaging=EvaluationAveraging.Macro):
        if isinstance(c, str):
            c, averaging = None, c
        if c is not None:
            return self._ratio(self.truePositives(c), self.truePositives(c) + self.falsePositives(c), edgeCase)
        return self._averaged(lambda i: self.precision(i), lambda i: self.truePositives(i) + self.falsePositives(i) > 0, averaging,
                              lambda: self._ratio(sum(self.truePositives().values()),
                                                  sum(self.truePositives().values()) + sum(self.falsePositives().values())))

    def recall(self, c=None, edgeCase=0.0, averaging=EvaluationAveraging.Macro):
        if isinstance(c, str):
            c, averaging = None, c
        if c is not None:
            return self._ratio(self.truePositives(c), self.truePositives(c) + self.falseNegatives(c), edgeCase)
        return self._averaged(lambda i: self.recall(i), lambda i: self.truePositives(i) + self.falseNegatives(i) > 0, averaging,
                              lambda: self._ratio(sum(self.truePositives().values()),
                                                  sum(self.truePositives().values()) + sum(self.falseNegatives().values())))

    def falsePositiveRate(self, c=None, edgeCase=0.0, averaging=EvaluationAveraging.Macro):
        if c is not None:
            return self._ratio(self.falsePositives(c), self.falsePositives(c) + self.trueNegatives(c), edgeCase)
        return self._averaged(lambda i: self.falsePositiveRate(i), lambda i: True, averaging,
                              lambda: self._ratio(sum(self.falsePositives().values()),
                                                  sum(self.falsePositives().values()) + sum(self.trueNegatives().values())))

    def falseNegativeRate(self, c=None, edgeCase=0.0, averaging=EvaluationAveraging.Macro):
        if c is not None:
            return self._ratio(self.falseNegatives(c), self.falseNegatives(c) + self.truePositives(c), edgeCase)
        return self._averaged(lambda i: self.falseNegativeRate(i), lambda i: True, averaging,
                              lambda: self._ratio(sum(self.falseNegatives().values()),
                                                  sum(self.falseNegatives().values()) + sum(self.truePositives().values())))

    def falseAlarmRate(self):
        return (self.falsePositiveRate() + self.falseNegativeRate()) / 2.0

    def fBeta(self, beta, c=None, defaultValue=0.0, averaging=EvaluationAveraging.Macro):
        if c is not None:
            p, r = self.precision(c), self.recall(c)
            if self.truePositives(c) + self.falsePositives(c) == 0 or self.truePositives(c) + self.falseNegatives(c) == 0:
                return defaultValue
            return self._ratio((1 + beta * beta) * p * r, beta * beta * p + r)
        def micro():
            tp, fp, fn = (sum(x.values()) for x in (self.truePositives(), self.falsePositives(), self.falseNegatives()))
            p, r = self._ratio(tp, tp + fp), self._ratio(tp, tp + fn)
            return self._ratio((1 + beta * beta) * p * r, beta * beta * p + r)
        return self._averaged(lambda i: self.fBeta(beta, i), lambda i: self.truePositives(i) + self.falsePositives(i) > 0 and
                              self.truePositives(i) + self.falseNegatives(i) > 0, averaging, micro)

    def f1(self, c=None, averaging=EvaluationAveraging.Macro):
        if isinstance(c, str):
            c, averaging = None, c
        return self.fBeta(1.0, c, averaging=averaging)

    def gMeasure(self, c=None, averaging=EvaluationAveraging.Macro):
        if c is not None:
            return math.sqrt(self.precision(c) * self.recall(c))
        return self._averaged(lambda i: self.gMeasure(i), lambda i: True, averaging,
                              lambda: math.sqrt(self.precision(averaging="Micro") * self.recall(averaging="Micro")))

    def matthewsCorrelation(self, c=None, averaging=EvaluationAveraging.Macro):
        if c is not None:
            tp, fp, fn, tn = self.truePositives(c), self.falsePositives(c), self.falseNegatives(c), self.trueNegatives(c)
            den = math.sqrt(float(tp + fp) * (tp + fn) * (tn + fp) * (tn + fn))
            return (tp * tn - fp * fn) / den if den else 0.0
        def micro():
            tp, fp, fn, tn = (sum(x.values()) for x in (self.truePositives(), self.falsePositives(), self.falseNegatives(), self.trueNegatives()))
            den = math.sqrt(float(tp + fp) * (tp + fn) * (tn + fp) * (tn + fn))
            return (tp * tn - fp * fn) / den if den else 0.0
        return self._averaged(lambda i: self.matthewsCorrelation(i), lambda i: True, averaging, micro)

    def scoreForMetric(self, metric):
        return {"ACCURACY": self.accuracy, "F1": self.f1, "PRECISION": self.precision, "RECALL": self.recall,
                "GMEASURE": self.gMeasure, "MCC": self.matthewsCorrelation}[str(metric).upper()]()

    def getValue(self, metric):
        return self.scoreForMetric(metric)

    # ------------------------------------------------------------------ reporting
    def _label(self, i):
        return self.labelsList[i] if self.labelsList and i < len(self.labelsList) else str(i)

    def stats(self, suppressWarnings=False, includeConfusion=True):
        if self.confusion_ is None:
            return "Evaluation: no data"
        n = self.numClasses
        lines = ["", "========================Evaluation Metrics========================",
                 f" # of classes:    {n}", f" Accuracy:        {self.accuracy():.4f}"]
        if self.topN > 1:
            lines.append(f" Top {self.topN} Accuracy:  {self.topNAccuracy():.4f}")
        lines += [f" Precision:       {self.precision():.4f}", f" Recall:          {self.recall():.4f}",
                  f" F1 Score:        {self.f1():.4f}"]
        if self._is_binary():
            lines.append(f"Precision, recall & F1: reported for positive class (class {self.binaryPositiveClass} - \"{self._label(self.binaryPositiveClass)}\") only")
        else:
            lines.append(f"Precision, recall & F1: macro-averaged (equally weighted avg. of {n} classes)")
            if not suppressWarnings:
                never = [self._label(i) for i in range(n) if self.truePositives(i) + self.falsePositives(i) == 0]
                if never:
                    lines.append(f"Warning: {len(never)} class(es) were never predicted by the model and were excluded from average precision: {never}")
        if includeConfusion:
            lines += ["", "=========================Confusion Matrix========================="]
            w = max(5, len(str(int(self._m().max()))) + 1)
            lines.append(" ".join(f"{i:>{w}}" for i in range(n)))
            lines.append("-" * ((w + 1) * n))
            for i in range(n):
                lines.append(" ".join(f"{int(v):>{w}}" for v in self._m()[i]) + f" | {i} = {self._label(i)}")
            lines += ["", "Confusion matrix format: Actual (rowClass) predicted as (columnClass) N times"]
        lines.append("==================================================================")
        return "\n".join(lines)

    def toJson(self):
        return json.dumps({"@class": "org.nd4j.evaluation.classification.Evaluation", "numClasses": self.numClasses, "topN": self.topN,
                           "labelsList": self.labelsList, "confusion": self._m().tolist(), "topNCorrectCount": self.topNCorrectCount,
                           "topNTotalCount": self.topNTotalCount, "numRowCounter": self.numRowCounter,
                           "binaryPositiveClass": self.binaryPositiveClass, "binaryDecisionThreshold": self.binaryDecisionThreshold})

    @staticmethod
    def fromJson(s):
        d = json.loads(s)
        e = Evaluation(d["numClasses"], d.get("labelsList"), d.get("topN", 1), d.get("binaryPositiveClass", 1), d.get("binaryDecisionThreshold"))
        if d.get("confusion"):
            e._ensure(d["numClasses"])
            e.confusion_.m = torch.tensor(d["confusion"], dtype=torch.int64)
        e.topNCorrectCount, e.topNTotalCount, e.numRowCounter = d["topNCorrectCount"], d["topNTotalCount"], d["numRowCounter"]
        return e

    def newInstance(self):
        return Evaluation(self.numClasses, self.labelsList, self.topN, self.binaryPositiveClass, self.binaryDecisionThreshold, self.costArray)


class EvaluationBinary:
    """Independent binary outputs (sigmoid per column); counts kept per output."""

    def __init__(self, size=None, rocBinarySteps=None, decisionThreshold=None):
        self.decisionThreshold = _t(decisionThreshold)
        self.tp = self.fp = self.tn = self.fn = None
        self.labels = None
        self.rocBinary = None
        if rocBinarySteps is not None:
            from .roc import ROCBinary
            self.rocBinary = ROCBinary(rocBinarySteps)

    def reset(self):
        self.tp = self.fp = self.tn = self.fn = None

    def eval(self, labels, predictions, mask=None, recordMetaData=None):
        labels, preds, mask = flatten_time_series(labels, predictions, mask)
        p = preds.float()
        thr = 0.5 if self.decisionThreshold is None else self.decisionThreshold.to(p.device).reshape(1, -1)
        guess = p > thr
        act = labels > 0.5
        w = torch.ones_like(p, dtype=torch.bool) if mask is None else (mask > 0).expand_as(p) if mask.dim() == 2 and mask.shape[1] == p.shape[1] else (mask.reshape(-1, 1) > 0).expand_as(p)
        def cnt(x):
            return (x & w).sum(0).cpu().long()
        vals = cnt(guess & act), cnt(guess & ~act), cnt(~guess & ~act), cnt(~guess & act)
        if self.tp is None:
            self.tp, self.fp, self.tn, self.fn = vals
        else:
            self.tp += vals[0]; self.fp += vals[1]; self.tn += vals[2]; self.fn += vals[3]
        if self.rocBinary is not None:
            self.rocBinary.eval(labels, preds, mask)

    def merge(self, o):
        if o.tp is None:
            return self
        if self.tp is None:
            self.tp, self.fp, self.tn, self.fn = o.tp.clone(), o.fp.clone(), o.tn.clone(), o.fn.clone()
        else:
            self.tp += o.tp; self.fp += o.fp; self.tn += o.tn; self.fn += o.fn
        return self

    def numLabels(self): return 0 if self.tp is None else self.tp.numel()
    def setLabelNames(self, names): self.labels = list(names)
    def truePositives(self, i): return int(self.tp[i])
    def falsePositives(self, i): return int(self.fp[i])
    def trueNegatives(self, i): return int(self.tn[i])
    def falseNegatives(self, i): return int(self.fn[i])
    def totalCount(self, i): return int(self.tp[i] + self.fp[i] + self.tn[i] + self.fn[i])
    def accuracy(self, i): return Evaluation._ratio(int(self.tp[i] + self.tn[i]), self.totalCount(i))
    def precision(self, i): return Evaluation._ratio(int(self.tp[i]), int(self.tp[i] + self.fp[i]))
    def recall(self, i): return Evaluation._ratio(int(self.tp[i]), int(self.tp[i] + self.fn[i]))
    def falsePositiveRate(self, i): return Evaluation._ratio(int(self.fp[i]), int(self.fp[i] + self.tn[i]))
    def falseNegativeRate(self, i): return Evaluation._ratio(int(self.fn[i]), int(self.fn[i] + self.tp[i]))

    def fBeta(self, beta, i):
        p, r = self.precision(i), self.recall(i)
        return Evaluation._ratio((1 + beta * beta) * p * r, beta * beta * p + r)

    def f1(self, i): return self.fBeta(1.0, i)

    def matthewsCorrelation(self, i):
        tp, fp, fn, tn = (int(x[i]) for x in (self.tp, self.fp, self.fn, self.tn))
        den = math.sqrt(float(tp + fp) * (tp + fn) * (tn + fp) * (tn + fn))
        return (tp * tn - fp * fn) / den if den else 0.0

    def gMeasure(self, i): return math.sqrt(self.precision(i) * self.recall(i))

    def _avg(self, fn): return sum(fn(i) for i in range(self.numLabels())) / max(self.numLabels(), 1)
    def averageAccuracy(self): return self._avg(self.accuracy)
    def averagePrecision(self): return self._avg(self.precision)
    def averageRecall(self): return self._avg(self.recall)
    def averageF1(self): return self._avg(self.f1)

    def scoreForMetric(self, metric, i):
        return {"ACCURACY": self.accuracy, "F1": self.f1, "PRECISION": self.precision, "RECALL": self.recall, "GMEASURE": self.gMeasure,
                "MCC": self.matthewsCorrelation, "FPR": self.falsePositiveRate, "FNR": self.falseNegativeRate}[str(metric).upper()](i)

    def stats(self, printPrecision=4):
        hdr = f"{'Label':<12}{'Accuracy':>10}{'F1':>10}{'Precision':>10}{'Recall':>10}{'Total':>8}{'TP':>7}{'TN':>7}{'FP':>7}{'FN':>7}"
        rows = [hdr]
        for i in range(self.numLabels()):
            nm = self.labels[i] if self.labels else f"label_{i}"
            rows.append(f"{nm:<12}{self.accuracy(i):>10.{printPrecision}f}{self.f1(i):>10.{printPrecision}f}{self.precision(i):>10.{printPrecision}f}"
                        f"{self.recall(i):>10.{printPrecision}f}{self.totalCount(i):>8}{int(self.tp[i]):>7}{int(self.tn[i]):>7}{int(self.fp[i]):>7}{int(self.fn[i]):>7}")
        return "\n".join(rows)


class EvaluationCalibration:
    def __init__(self, reliabilityDiagNumBins=10, histogramNumBins=50, excludeEmptyBins=True):
        self.rBins, self.hBins, self.excludeEmptyBins = reliabilityDiagNumBins, histogramNumBins, excludeEmptyBins
        self.rCounts = self.rPos = self.rSumP = None
        self.labelCounts = self.predCounts = None
        self.residOverall = self.residByLabel = self.probOverall = self.probByLabel = None

    def eval(self, labels, predictions, mask=None, recordMetaData=None):
        labels, preds, mask = flatten_time_series(labels, predictions, mask)
        p, l = preds.float(), labels.float()
        n, c = p.shape
        if self.rCounts is None:
            z = lambda *s: torch.zeros(*s, dtype=torch.float64)
            self.rCounts, self.rPos, self.rSumP = z(c, self.rBins), z(c, self.rBins), z(c, self.rBins)
            self.labelCounts, self.predCounts = z(c), z(c)
            self.residOverall, self.residByLabel = z(self.hBins), z(c, self.hBins)
            self.probOverall, self.probByLabel = z(self.hBins), z(c, self.hBins)
        bins = (p * self.rBins).long().clamp_(0, self.rBins - 1)
        cls = torch.arange(c, device=p.device).expand(n, c)
        flat = (cls * self.rBins + bins).reshape(-1)
        def acc(dst, w):
            dst += torch.bincount(flat, weights=w.reshape(-1).double(), minlength=c * self.rBins).reshape(c, self.rBins).cpu()
        acc(self.rCounts, torch.ones_like(p)); acc(self.rPos, l); acc(self.rSumP, p)
        self.labelCounts += l.sum(0).double().cpu()
        self.predCounts += torch.bincount(p.argmax(1), minlength=c).double().cpu()
        resid = (l - p).abs()
        hb = (resid * self.hBins).long().clamp_(0, self.hBins - 1)
        pb = (p * self.hBins).long().clamp_(0, self.hBins - 1)
        self.residOverall += torch.bincount(hb.reshape(-1), minlength=self.hBins).double().cpu()
        self.probOverall += torch.bincount(pb.reshape(-1), minlength=self.hBins).double().cpu()
        is_lab = l > 0.5
        for dst, b in ((self.residByLabel, hb), (self.probByLabel, pb)):
            f = (cls * self.hBins + b)[is_lab]
            dst += torch.bincount(f, minlength=c * self.hBins).reshape(c, self.hBins).double().cpu()

    def merge(self, o):
        if o.rCounts is None:
            return self
        if self.rCounts is None:
            self.__dict__.update({k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in o.__dict__.items()})
            return self
        for k in ("rCounts", "rPos", "rSumP", "labelCounts", "predCounts", "residOverall", "residByLabel", "probOverall", "probByLabel"):
            getattr(self, k).add_(getattr(o, k))
        return self

    def getReliabilityDiagram(self, classIdx):
        cnt, pos, sp = self.rCounts[classIdx], self.rPos[classIdx], self.rSumP[classIdx]
        keep = cnt > 0 if self.excludeEmptyBins else torch.ones_like(cnt, dtype=torch.bool)
        safe = cnt.clamp(min=1)
        return {"title": f"Reliability Diagram: Class {classIdx}", "meanPredictedValueX": (sp / safe)[keep].tolist(),
                "fractionPositivesY": (pos / safe)[keep].tolist()}

    def expectedCalibrationError(self, classIdx):
        cnt, pos, sp = self.rCounts[classIdx], self.rPos[classIdx], self.rSumP[classIdx]
        tot = float(cnt.sum())
        safe = cnt.clamp(min=1)
        return float(((pos / safe - sp / safe).abs() * cnt).sum() / tot) if tot else 0.0

    def getLabelCountsEachClass(self): return self.labelCounts.long().tolist()
    def getPredictionCountsEachClass(self): return self.predCounts.long().tolist()
    def getResidualPlotAllClasses(self): return {"binCounts": self.residOverall.long().tolist(), "lower": 0.0, "upper": 1.0}
    def getResidualPlot(self, c): return {"binCounts": self.residByLabel[c].long().tolist(), "lower": 0.0, "upper": 1.0}
    def getProbabilityHistogramAllClasses(self): return {"binCounts": self.probOverall.long().tolist(), "lower": 0.0, "upper": 1.0}
    def getProbabilityHistogram(self, c): return {"binCounts": self.probByLabel[c].long().tolist(), "lower": 0.0, "upper": 1.0}

    def stats(self):
        return f"EvaluationCalibration(nBins={self.rBins}, numClasses={0 if self.rCounts is None else self.rCounts.shape[0]})"
