"""Early stopping (``deeplearning4j-nn/.../earlystopping``): configuration, termination conditions,
score calculators, model savers, trainer and result."""
from __future__ import annotations

import math
import os
import time


# ----------------------------------------------------------------------------- termination conditions
class EpochTerminationCondition:
    def initialize(self): pass
    def terminate(self, epochNum, score, minimize): raise NotImplementedError


class MaxEpochsTerminationCondition(EpochTerminationCondition):
    def __init__(self, maxEpochs): self.maxEpochs = int(maxEpochs)
    def terminate(self, epochNum, score, minimize): return epochNum + 1 >= self.maxEpochs
    def __repr__(self): return f"MaxEpochsTerminationCondition({self.maxEpochs})"


class ScoreImprovementEpochTerminationCondition(EpochTerminationCondition):
    """Stop after ``maxEpochsWithNoImprovement`` epochs without an improvement of at least ``minImprovement``."""

    def __init__(self, maxEpochsWithNoImprovement, minImprovement=0.0):
        self.maxNoImprove, self.minImprovement = int(maxEpochsWithNoImprovement), float(minImprovement)

    def initialize(self):
        self.bestExpectedScore, self.bestEpoch = None, -1

    def terminate(self, epochNum, score, minimize):
        if self.bestExpectedScore is None:
            self.bestExpectedScore, self.bestEpoch = score, epochNum
            return False
        improvement = (self.bestExpectedScore - score) if minimize else (score - self.bestExpectedScore)
        if improvement > self.minImprovement:
            self.bestExpectedScore, self.bestEpoch = score, epochNum
            return False
        return epochNum >= self.bestEpoch + self.maxNoImprove

    def __repr__(self): return f"ScoreImprovementEpochTerminationCondition(maxEpochsWithNoImprovement={self.maxNoImprove}, minImprovement={self.minImprovement})"


class BestScoreEpochTerminationCondition(EpochTerminationCondition):
    def __init__(self, bestExpectedScore): self.best = float(bestExpectedScore)
    def terminate(self, epochNum, score, minimize): return score < self.best if minimize else score > self.best
    def __repr__(self): return f"BestScoreEpochTerminationCondition({self.best})"


class IterationTerminationCondition:
    def initialize(self): pass
    def terminate(self, lastMiniBatchScore): raise NotImplementedError


class MaxTimeIterationTerminationCondition(IterationTerminationCondition):
    def __init__(self, maxTimeAmount, unit="seconds"):
        mult = {"ms": 1e-3, "milliseconds": 1e-3, "s": 1, "seconds": 1, "minutes": 60, "hours": 3600}[str(unit).lower()]
        self.maxSeconds = maxTimeAmount * mult

    def initialize(self): self.start = time.time()
    def terminate(self, lastMiniBatchScore): return time.time() - self.start >= self.maxSeconds
    def __repr__(self): return f"MaxTimeIterationTerminationCondition({self.maxSeconds}s)"


class MaxScoreIterationTerminationCondition(IterationTerminationCondition):
    def __init__(self, maxScore): self.maxScore = float(maxScore)
    def terminate(self, s): return s > self.maxScore
    def __repr__(self): return f"MaxScoreIterationTerminationCondition({self.maxScore})"


class InvalidScoreIterationTerminationCondition(IterationTerminationCondition):
    def terminate(self, s): return math.isnan(s) or math.isinf(s)
    def __repr__(self): return "InvalidScoreIterationTerminationCondition()"


# ----------------------------------------------------------------------------- score calculators
class ScoreCalculator:
    def calculateScore(self, net): raise NotImplementedError
    def minimizeScore(self): return True


class DataSetLossCalculator(ScoreCalculator):
    """Average (or summed) loss over an iterator."""

    def __init__(self, iterator, average=True):
        self.iterator, self.average = iterator, average

    def calculateScore(self, net):
        if hasattr(self.iterator, "reset"):
            self.iterator.reset()
        tot, n = 0.0, 0
        for ds in self.iterator:
            b = ds.numExamples() if hasattr(ds, "numExamples") else 1
            tot += float(net.score(ds)) * b
            n += b
        return tot / n if self.average and n else tot


class ClassificationScoreCalculator(ScoreCalculator):
    def __init__(self, metric, iterator): self.metric, self.iterator = metric, iterator
    def calculateScore(self, net): return net.evaluate(self.iterator).scoreForMetric(self.metric)
    def minimizeScore(self): return False


class RegressionScoreCalculator(ScoreCalculator):
    def __init__(self, metric, iterator): self.metric, self.iterator = metric, iterator
    def calculateScore(self, net): return net.evaluateRegression(self.iterator).scoreForMetric(self.metric)
    def minimizeScore(self): return str(self.metric).upper() not in ("R2", "PC")


class ROCScoreCalculator(ScoreCalculator):
    def __init__(self, rocType, metric_or_iter, iterator=None):
        self.rocType = rocType
        self.metric, self.iterator = ("AUROC", metric_or_iter) if iterator is None else (metric_or_iter, iterator)

    def calculateScore(self, net):
        from ..eval import ROC, ROCBinary, ROCMultiClass
        ev = {"ROC": ROC, "BINARY": ROCBinary, "MULTICLASS": ROCMultiClass}[str(self.rocType).upper()](0)
        net.doEvaluation(self.iterator, ev)
        return ev.scoreForMetric(self.metric)

    def minimizeScore(self): return False


class AutoencoderScoreCalculator(ScoreCalculator):
    """Reconstruction error of an AutoEncoder layer (layer 0) over an iterator."""

    def __init__(self, metric, iterator): self.metric, self.iterator = metric, iterator

    def calculateScore(self, net):
        from ..eval import RegressionEvaluation
        ev = RegressionEvaluation()
        if hasattr(self.iterator, "reset"):
            self.iterator.reset()
        for ds in self.iterator:
            x = ds.getFeatures()
            ev.eval(x, net.output(x))
        return ev.scoreForMetric(self.metric)


# ----------------------------------------------------------------------------- savers
class InMemoryModelSaver:
    def __init__(self): self.best = self.latest = None
    def saveBestModel(self, net, score): self.best = net.clone()
    def saveLatestModel(self, net, score): self.latest = net.clone()
    def getBestModel(self): return self.best
    def getLatestModel(self): return self.latest


class LocalFileModelSaver:
    """``bestModel.bin`` / ``latestModel.bin`` in a directory (ModelSerializer zip format)."""

    def __init__(self, directory):
        self.directory = str(directory)
        os.makedirs(self.directory, exist_ok=True)

    def _path(self, which): return os.path.join(self.directory, f"{which}Model.bin")

    def saveBestModel(self, net, score):
        from .serializer import ModelSerializer
        ModelSerializer.writeModel(net, self._path("best"), True)

    def saveLatestModel(self, net, score):
        from .serializer import ModelSerializer
        ModelSerializer.writeModel(net, self._path("latest"), True)

    def _load(self, which):
        from .serializer import ModelGuesser
        p = self._path(which)
        return ModelGuesser.loadModelGuess(p) if os.path.exists(p) else None

    def getBestModel(self): return self._load("best")
    def getLatestModel(self): return self._load("latest")


LocalFileGraphSaver = LocalFileModelSaver


# ----------------------------------------------------------------------------- configuration / result / trainer
class EarlyStoppingConfiguration:
    def __init__(self, epochTerminationConditions=None, iterationTerminationConditions=None, scoreCalculator=None,
                 evaluateEveryNEpochs=1, modelSaver=None, saveLastModel=False):
        self.epochTerminationConditions = list(epochTerminationConditions or [])
        self.iterationTerminationConditions = list(iterationTerminationConditions or [])
        self.scoreCalculator, self.evaluateEveryNEpochs = scoreCalculator, max(int(evaluateEveryNEpochs), 1)
        self.modelSaver, self.saveLastModel = modelSaver or InMemoryModelSaver(), saveLastModel

    class Builder:
        def __init__(self): self.kw = {}
        def epochTerminationConditions(self, *c): self.kw["epochTerminationConditions"] = list(c[0]) if len(c) == 1 and isinstance(c[0], (list, tuple)) else list(c); return self
        def iterationTerminationConditions(self, *c): self.kw["iterationTerminationConditions"] = list(c[0]) if len(c) == 1 and isinstance(c[0], (list, tuple)) else list(c); return self
        def scoreCalculator(self, s): self.kw["scoreCalculator"] = s; return self
        def evaluateEveryNEpochs(self, n): self.kw["evaluateEveryNEpochs"] = n; return self
        def modelSaver(self, s): self.kw["modelSaver"] = s; return self
        def saveLastModel(self, b): self.kw["saveLastModel"] = b; return self
        def build(self): return EarlyStoppingConfiguration(**self.kw)


class TerminationReason:
    Error = "Error"
    IterationTerminationCondition = "IterationTerminationCondition"
    EpochTerminationCondition = "EpochTerminationCondition"


class EarlyStoppingResult:
    def __init__(self, terminationReason, terminationDetails, scoreVsEpoch, bestModelEpoch, bestModelScore, totalEpochs, bestModel):
        self.terminationReason, self.terminationDetails, self.scoreVsEpoch = terminationReason, terminationDetails, scoreVsEpoch
        self.bestModelEpoch, self.bestModelScore, self.totalEpochs, self.bestModel = bestModelEpoch, bestModelScore, totalEpochs, bestModel

    def getTerminationReason(self): return self.terminationReason
    def getTerminationDetails(self): return self.terminationDetails
    def getScoreVsEpoch(self): return self.scoreVsEpoch
    def getBestModelEpoch(self): return self.bestModelEpoch
    def getBestModelScore(self): return self.bestModelScore
    def getTotalEpochs(self): return self.totalEpochs
    def getBestModel(self): return self.bestModel

    def __repr__(self):
        return (f"EarlyStoppingResult(terminationReason={self.terminationReason},details={self.terminationDetails},"
                f"bestModelEpoch={self.bestModelEpoch},bestModelScore={self.bestModelScore},totalEpochs={self.totalEpochs})")


class EarlyStoppingListener:
    def onStart(self, esConfig, net): pass
    def onEpoch(self, epochNum, score, esConfig, net): pass
    def onCompletion(self, esResult): pass


class EarlyStoppingTrainer:
    """``trainer/BaseEarlyStoppingTrainer.java``: epoch loop with per-iteration and per-epoch stop checks.
    The per-iteration check reads the mini-batch score, which synchronises with the device; it is skipped when
    no iteration termination conditions are configured."""

    def __init__(self, esConfig, net, train, listener=None):
        self.esConfig, self.net, self.train, self.listener = esConfig, net, train, listener

    def setListener(self, l): self.listener = l

    def fit(self):
        es, net = self.esConfig, self.net
        for c in es.epochTerminationConditions + es.iterationTerminationConditions:
            c.initialize()
        if self.listener:
            self.listener.onStart(es, net)
        scoreVsEpoch = {}
        minimize = es.scoreCalculator.minimizeScore() if es.scoreCalculator else True
        best_score, best_epoch = (math.inf if minimize else -math.inf), -1
        epoch = 0
        reason, details = None, None
        while True:
            if hasattr(self.train, "reset"):
                self.train.reset()
            stop_iter = None
            try:
                for ds in self.train:
                    net.fit(ds)
                    if es.iterationTerminationConditions:
                        s = float(net.score())
                        for c in es.iterationTerminationConditions:
                            if c.terminate(s):
                                stop_iter = c
                                break
                    if stop_iter is not None:
                        break
            except Exception as e:                          # noqa: BLE001 - reported through the result like the reference
                reason, details = TerminationReason.Error, repr(e)
                break
            if stop_iter is not None:
                reason, details = TerminationReason.IterationTerminationCondition, repr(stop_iter)
                if es.saveLastModel:
                    es.modelSaver.saveLatestModel(net, 0.0)
                break
            net.incrementEpochCount()
            if epoch % es.evaluateEveryNEpochs == 0 or epoch == 0:
                score = es.scoreCalculator.calculateScore(net) if es.scoreCalculator else float(net.score())
                scoreVsEpoch[epoch] = score
                if (minimize and score < best_score) or (not minimize and score > best_score):
                    best_score, best_epoch = score, epoch
                    es.modelSaver.saveBestModel(net, score)
                if es.saveLastModel:
                    es.modelSaver.saveLatestModel(net, score)
                if self.listener:
                    self.listener.onEpoch(epoch, score, es, net)
                stop = next((c for c in es.epochTerminationConditions if c.terminate(epoch, score, minimize)), None)
            else:
                stop = next((c for c in es.epochTerminationConditions if isinstance(c, MaxEpochsTerminationCondition)
                             and c.terminate(epoch, 0.0, minimize)), None)
            if stop is not None:
                reason, details = TerminationReason.EpochTerminationCondition, repr(stop)
                epoch += 1
                break
            epoch += 1
        best = es.modelSaver.getBestModel()
        res = EarlyStoppingResult(reason, details, scoreVsEpoch, best_epoch, best_score, epoch, best)
        if self.listener:
            self.listener.onCompletion(res)
        return res


EarlyStoppingGraphTrainer = EarlyStoppingTrainer
