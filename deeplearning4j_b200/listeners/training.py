"""DL4J training listeners (``deeplearning4j-nn/.../optimize/listeners``).

The networks call ``iterationDone(model, iteration, epoch)``, ``onEpochStart(model)``,
``onEpochEnd(model)``, ``onForwardPass``, ``onGradientCalculation`` and ``onBackwardPass`` on every
attached listener.  Listeners that only need a number now and then (score printing, throughput)
avoid a device synchronisation on the iterations they skip: ``model.score()`` is only read when the
report is actually due.
"""
from __future__ import annotations

import getpass
import logging
import os
import random
import socket
import sys
import time

log = logging.getLogger("deeplearning4j_b200")


class TrainingListener:
    def iterationDone(self, model, iteration, epoch): pass
    def onEpochStart(self, model): pass
    def onEpochEnd(self, model): pass
    def onForwardPass(self, model, activations=None): pass
    def onGradientCalculation(self, model): pass
    def onBackwardPass(self, model): pass


BaseTrainingListener = TrainingListener


class ScoreIterationListener(TrainingListener):
    """``ScoreIterationListener.java``: logs the score every ``printIterations`` iterations."""

    def __init__(self, printIterations=10, out=None):
        self.printIterations = max(int(printIterations), 1)
        self.out = out

    def iterationDone(self, model, iteration, epoch):
        if iteration % self.printIterations == 0:
            msg = f"Score at iteration {iteration} is {model.score()}"
            (self.out or log.info)(msg) if self.out is None else print(msg, file=self.out)


class PerformanceListener(TrainingListener):
    """``PerformanceListener.java:139,250``: iteration time, samples/sec, batches/sec, ETL time, score."""

    def __init__(self, frequency=1, reportScore=False, reportGC=False, reportSample=True, reportBatch=True, reportIteration=True,
                 reportEtl=True, reportTime=True, out=None):
        self.frequency = max(int(frequency), 1)
        self.reportScore, self.reportSample, self.reportBatch = reportScore, reportSample, reportBatch
        self.reportIteration, self.reportEtl, self.reportTime = reportIteration, reportEtl, reportTime
        self.out = out
        self._last = None
        self._samples = 0
        self._batches = 0
        self.samplesPerSec = self.batchesPerSec = 0.0
        self.lastMessage = None

    class Builder:
        def __init__(self): self.kw = {}
        def reportScore(self, b): self.kw["reportScore"] = b; return self
        def reportSample(self, b): self.kw["reportSample"] = b; return self
        def reportBatch(self, b): self.kw["reportBatch"] = b; return self
        def reportIteration(self, b): self.kw["reportIteration"] = b; return self
        def reportETL(self, b): self.kw["reportEtl"] = b; return self
        def reportTime(self, b): self.kw["reportTime"] = b; return self
        def setFrequency(self, f): self.kw["frequency"] = f; return self
        def build(self): return PerformanceListener(**self.kw)

    def iterationDone(self, model, iteration, epoch):
        now = time.perf_counter()
        if self._last is None:
            self._last = now
        self._samples += int(getattr(model, "_last_batch", 0) or 0)
        self._batches += 1
        if iteration % self.frequency != 0 or self._batches == 0:
            return
        if self.reportScore:
            score = model.score()                      # synchronises: time after it so throughput includes the device work
            now = time.perf_counter()
        dt = max(now - self._last, 1e-9)
        self.samplesPerSec, self.batchesPerSec = self._samples / dt, self._batches / dt
        parts = []
        if self.reportEtl:
            parts.append(f"ETL: {int(getattr(model, '_last_etl_ms', 0) or 0)} ms; ")
        if self.reportIteration:
            parts.append(f"iteration {iteration}; ")
        if self.reportTime:
            parts.append(f"iteration time: {int(dt * 1e3 / self._batches)} ms; ")
        if self.reportSample:
            parts.append(f"samples/sec: {self.samplesPerSec:.3f}; ")
        if self.reportBatch:
            parts.append(f"batches/sec: {self.batchesPerSec:.3f}; ")
        if self.reportScore:
            parts.append(f"score: {score};")
        self.lastMessage = "".join(parts)
        log.info(self.lastMessage) if self.out is None else print(self.lastMessage, file=self.out)
        self._last, self._samples, self._batches = time.perf_counter(), 0, 0


class CollectScoresIterationListener(TrainingListener):
    def __init__(self, frequency=1):
        self.frequency = max(int(frequency), 1)
        self.scoreVsIter = []

    def iterationDone(self, model, iteration, epoch):
        if iteration % self.frequency == 0:
            self.scoreVsIter.append((iteration, model.score()))

    def getScoreVsIter(self): return self.scoreVsIter

    def exportScores(self, path, delimiter=","):
        with open(path, "w") as f:
            f.write(f"Iteration{delimiter}Score\n")
            for i, s in self.scoreVsIter:
                f.write(f"{i}{delimiter}{s}\n")


class CollectScoresListener(CollectScoresIterationListener):
    def __init__(self, frequency=1, logScore=False):
        super().__init__(frequency)
        self.logScore = logScore

    def iterationDone(self, model, iteration, epoch):
        super().iterationDone(model, iteration, epoch)
        if self.logScore and iteration % self.frequency == 0:
            log.info("Score at iteration %d is %s", iteration, self.scoreVsIter[-1][1])

    def getListIteration(self): return [i for i, _ in self.scoreVsIter]
    def getListScore(self): return [s for _, s in self.scoreVsIter]


class TimeIterationListener(TrainingListener):
    """Estimates the remaining training time from the iterations done so far."""

    def __init__(self, iterationCount, frequency=1):
        self.iterationCount, self.frequency = int(iterationCount), max(int(frequency), 1)
        self.start = time.time()
        self.counter = 0
        self.lastMessage = None

    def iterationDone(self, model, iteration, epoch):
        self.counter += 1
        if self.counter % self.frequency:
            return
        elapsed = time.time() - self.start
        remaining = elapsed / self.counter * max(self.iterationCount - self.counter, 0)
        self.lastMessage = f"Remaining time : {int(remaining // 60)}mn - End expected : {time.ctime(time.time() + remaining)}"
        log.info(self.lastMessage)


class SleepyTrainingListener(TrainingListener):
    """Sleeps in the chosen callbacks (used to simulate slow workers)."""

    def __init__(self, timerEE=0, timerES=0, timerFF=0, timerBP=0, timerIteration=0, sleepMode="PARK"):
        self.timerEE, self.timerES, self.timerFF, self.timerBP, self.timerIteration = timerEE, timerES, timerFF, timerBP, timerIteration
        self.sleepMode = sleepMode

    def _sleep(self, ms):
        if ms > 0:
            time.sleep(ms / 1e3)

    def onEpochStart(self, model): self._sleep(self.timerES)
    def onEpochEnd(self, model): self._sleep(self.timerEE)
    def onForwardPass(self, model, activations=None): self._sleep(self.timerFF)
    def onBackwardPass(self, model): self._sleep(self.timerBP)
    def iterationDone(self, model, iteration, epoch): self._sleep(self.timerIteration)


class ComposableIterationListener(TrainingListener):
    def __init__(self, *listeners):
        self.listeners = list(listeners[0]) if len(listeners) == 1 and isinstance(listeners[0], (list, tuple)) else list(listeners)

    def iterationDone(self, model, iteration, epoch):
        for l in self.listeners:
            l.iterationDone(model, iteration, epoch)


class InvocationType:
    ITERATION_END = "ITERATION_END"
    EPOCH_END = "EPOCH_END"
    EPOCH_START = "EPOCH_START"


class EvaluativeListener(TrainingListener):
    """``EvaluativeListener.java``: runs evaluations on a held-out iterator every ``frequency`` invocations."""

    def __init__(self, iterator, frequency=1, invocationType=InvocationType.ITERATION_END, *evaluations):
        from ..eval import Evaluation
        self.iterator, self.frequency, self.invocationType = iterator, max(int(frequency), 1), invocationType
        self.evaluations = list(evaluations) or [Evaluation()]
        self.callback = None
        self.invocationCount = 0
        self.lastStats = None

    def setCallback(self, cb): self.callback = cb
    def getEvaluations(self): return self.evaluations

    def _invoke(self, model):
        self.invocationCount += 1
        if self.invocationCount % self.frequency:
            return
        for e in self.evaluations:
            e.reset()
        model.doEvaluation(self.iterator, *self.evaluations)
        self.lastStats = [e.stats() for e in self.evaluations]
        for s in self.lastStats:
            log.info("%s", s)
        if self.callback is not None:
            self.callback(self, model, self.invocationCount, self.evaluations)

    def iterationDone(self, model, iteration, epoch):
        if self.invocationType == InvocationType.ITERATION_END:
            self._invoke(model)

    def onEpochStart(self, model):
        if self.invocationType == InvocationType.EPOCH_START:
            self._invoke(model)

    def onEpochEnd(self, model):
        if self.invocationType == InvocationType.EPOCH_END:
            self._invoke(model)


# ----------------------------------------------------------------------------- checkpoints
class Checkpoint:
    HEADER = "checkpointNum,timestamp,iteration,epoch,modelType,filename"

    def __init__(self, checkpointNum, timestamp, iteration, epoch, modelType, filename):
        self.checkpointNum, self.timestamp, self.iteration, self.epoch = int(checkpointNum), int(timestamp), int(iteration), int(epoch)
        self.modelType, self.filename = modelType, filename

    def toFileString(self):
        return f"{self.checkpointNum},{self.timestamp},{self.iteration},{self.epoch},{self.modelType},{self.filename}"

    @staticmethod
    def fromFileString(s):
        parts = s.strip().split(",")
        if len(parts) != 6:
            raise ValueError(f"Cannot parse checkpoint entry: expected 6 entries, got {len(parts)} - values = {parts}")
        return Checkpoint(*parts)

    getCheckpointNum = lambda self: self.checkpointNum
    getFilename = lambda self: self.filename


class CheckpointListener(TrainingListener):
    """``CheckpointListener.java:40-300``: periodic ``checkpoint_<n>_<ModelType>.zip`` files plus a
    ``checkpointInfo.txt`` index; retention keep-all / keep-last-N / keep-last-N-and-every-M."""

    def __init__(self, rootDir, saveEveryNIterations=None, saveEveryNEpochs=None, saveEveryMs=None, saveEverySinceLast=True,
                 keepMode="ALL", keepLast=0, keepEvery=0, logSaving=True, deleteExisting=False, saveUpdater=True, continueExisting=False):
        self.rootDir = str(rootDir)
        os.makedirs(self.rootDir, exist_ok=True)
        self.saveEveryNIterations, self.saveEveryNEpochs, self.saveEveryMs = saveEveryNIterations, saveEveryNEpochs, saveEveryMs
        self.saveEverySinceLast = saveEverySinceLast
        self.keepMode, self.keepLast, self.keepEvery = keepMode, keepLast, keepEvery
        self.logSaving, self.saveUpdater = logSaving, saveUpdater
        self.recordFile = os.path.join(self.rootDir, "checkpointInfo.txt")
        existing = [f for f in os.listdir(self.rootDir) if f.startswith("checkpoint_") and f.endswith((".zip", "checkpointInfo.txt"))]
        if deleteExisting:
            for f in existing + (["checkpointInfo.txt"] if os.path.exists(self.recordFile) else []):
                p = os.path.join(self.rootDir, f)
                if os.path.exists(p):
                    os.remove(p)
        elif any(f.endswith(".zip") for f in existing) and not continueExisting:
            raise ValueError(f"Checkpoint directory {self.rootDir} already holds checkpoints; use deleteExisting(true) or another directory")
        self.checkpoints = []
        self.lastCheckpointNum = -1
        if continueExisting and os.path.exists(self.recordFile):
            # a resumed job keeps numbering (and pruning) where the previous one stopped
            self.checkpoints = CheckpointListener.availableCheckpoints(self.rootDir)
            self.lastCheckpointNum = max((c.checkpointNum for c in self.checkpoints), default=-1)
        self.startTime = self.lastSaveTime = None
        self.startIter = None

    class Builder:
        def __init__(self, rootDir): self.kw = {"rootDir": rootDir}
        def saveEveryNIterations(self, n): self.kw["saveEveryNIterations"] = n; return self
        saveEveryIteration = lambda self: self.saveEveryNIterations(1)
        def saveEveryNEpochs(self, n): self.kw["saveEveryNEpochs"] = n; return self
        saveEveryEpoch = lambda self: self.saveEveryNEpochs(1)
        def saveEvery(self, amount, unit="ms", sinceLast=True):
            mult = {"ms": 1, "s": 1e3, "sec": 1e3, "seconds": 1e3, "m": 6e4, "min": 6e4, "minutes": 6e4, "h": 3.6e6, "hours": 3.6e6}[str(unit).lower()]
            self.kw["saveEveryMs"], self.kw["saveEverySinceLast"] = amount * mult, sinceLast
            return self
        def keepAll(self): self.kw["keepMode"] = "ALL"; return self
        def keepLast(self, n): self.kw["keepMode"], self.kw["keepLast"] = "LAST", n; return self
        def keepLastAndEvery(self, n, every): self.kw.update(keepMode="LAST_AND_EVERY", keepLast=n, keepEvery=every); return self
        def logSaving(self, b): self.kw["logSaving"] = b; return self
        def deleteExisting(self, b): self.kw["deleteExisting"] = b; return self
        def saveUpdater(self, b): self.kw["saveUpdater"] = b; return self
        def continueExisting(self, b=True): self.kw["continueExisting"] = b; return self
        def build(self):
            if not any(self.kw.get(k) for k in ("saveEveryNIterations", "saveEveryNEpochs", "saveEveryMs")):
                raise ValueError("Cannot construct listener: no models will be saved (must use at least one of: save every N iter, N epochs or time)")
            return CheckpointListener(**self.kw)

    @staticmethod
    def builder(rootDir): return CheckpointListener.Builder(rootDir)

    def iterationDone(self, model, iteration, epoch):
        now = time.time()
        if self.startTime is None:
            self.startTime = self.lastSaveTime = now
            self.startIter = iteration
            return
        if self.saveEveryNIterations and iteration > 0 and iteration % self.saveEveryNIterations == 0:
            self._save(model, iteration, epoch)
        elif self.saveEveryMs:
            ref = self.lastSaveTime if self.saveEverySinceLast else self.startTime
            if (now - ref) * 1e3 >= self.saveEveryMs:
                self._save(model, iteration, epoch)
                if not self.saveEverySinceLast:
                    self.startTime = now

    def onEpochEnd(self, model):
        e = model.getEpochCount() + 1
        if self.saveEveryNEpochs and e > 0 and e % self.saveEveryNEpochs == 0:
            self._save(model, model.getIterationCount(), model.getEpochCount())

    @staticmethod
    def _file_name(num, modelType): return f"checkpoint_{num}_{modelType}.zip"

    def _save(self, model, iteration, epoch):
        from ..nn.serializer import ModelSerializer
        self.lastCheckpointNum += 1
        mt = type(model).__name__
        fn = self._file_name(self.lastCheckpointNum, mt)
        ModelSerializer.writeModel(model, os.path.join(self.rootDir, fn), self.saveUpdater)
        c = Checkpoint(self.lastCheckpointNum, int(time.time() * 1e3), iteration, epoch, mt, fn)
        new_file = not os.path.exists(self.recordFile)
        with open(self.recordFile, "a") as f:
            if new_file:
                f.write(Checkpoint.HEADER + "\n")
            f.write(c.toFileString() + "\n")
        self.checkpoints.append(c)
        self.lastSaveTime = time.time()
        if self.logSaving:
            log.info("Model checkpoint saved: epoch %d, iteration %d, path: %s", epoch, iteration, os.path.join(self.rootDir, fn))
        if self.keepMode != "ALL":
            keep = set(x.checkpointNum for x in self.checkpoints[-self.keepLast:]) if self.keepLast else set()
            for x in list(self.checkpoints):
                if x.checkpointNum in keep or (self.keepMode == "LAST_AND_EVERY" and self.keepEvery and x.checkpointNum % self.keepEvery == 0):
                    continue
                p = os.path.join(self.rootDir, x.filename)
                if os.path.exists(p):
                    os.remove(p)
                self.checkpoints.remove(x)

    # -- static helpers (directory based)
    @staticmethod
    def availableCheckpoints(directory=None):
        directory = directory.rootDir if isinstance(directory, CheckpointListener) else directory
        rec = os.path.join(directory, "checkpointInfo.txt")
        if not os.path.exists(rec):
            raise FileNotFoundError(f"Could not find checkpoint record file: {rec}")
        out = []
        with open(rec) as f:
            for line in list(f)[1:]:
                if line.strip():
                    c = Checkpoint.fromFileString(line)
                    if os.path.exists(os.path.join(directory, c.filename)):
                        out.append(c)
        return out

    def lastCheckpoint(self):
        a = CheckpointListener.availableCheckpoints(self.rootDir)
        return a[-1] if a else None

    @staticmethod
    def lastCheckpointIn(directory):
        a = CheckpointListener.availableCheckpoints(directory)
        return a[-1] if a else None

    @staticmethod
    def loadCheckpoint(directory, num_or_cp, loadUpdater=True):
        from ..nn.serializer import ModelGuesser
        cps = CheckpointListener.availableCheckpoints(directory)
        n = num_or_cp.checkpointNum if isinstance(num_or_cp, Checkpoint) else int(num_or_cp)
        for c in cps:
            if c.checkpointNum == n:
                return ModelGuesser.loadModelGuess(os.path.join(directory, c.filename))
        raise FileNotFoundError(f"checkpoint {n} not found in {directory}")

    loadCheckpointMLN = loadCheckpoint
    loadCheckpointCG = loadCheckpoint

    @staticmethod
    def loadLastCheckpoint(directory):
        c = CheckpointListener.lastCheckpointIn(directory)
        return None if c is None else CheckpointListener.loadCheckpoint(directory, c)

    loadLastCheckpointMLN = loadLastCheckpoint
    loadLastCheckpointCG = loadLastCheckpoint


# ----------------------------------------------------------------------------- failure injection (host side only)
class FailureMode:
    OOM = "OOM"
    SYSTEM_EXIT_1 = "SYSTEM_EXIT_1"
    ILLEGAL_STATE = "ILLEGAL_STATE"
    INFINITE_SLEEP = "INFINITE_SLEEP"


class CallType:
    ANY = "ANY"
    EPOCH_START = "EPOCH_START"
    EPOCH_END = "EPOCH_END"
    FORWARD_PASS = "FORWARD_PASS"
    GRADIENT_CALC = "GRADIENT_CALC"
    BACKWARD_PASS = "BACKWARD_PASS"
    ITER_DONE = "ITER_DONE"


class FailureTrigger:
    def initialize(self): pass
    def triggerFailure(self, callType, iteration, epoch, model): raise NotImplementedError


class And(FailureTrigger):
    def __init__(self, *triggers): self.triggers = list(triggers)
    def initialize(self): [t.initialize() for t in self.triggers]
    def triggerFailure(self, *a): return all(t.triggerFailure(*a) for t in self.triggers)


class Or(And):
    def triggerFailure(self, *a): return any(t.triggerFailure(*a) for t in self.triggers)


class RandomProb(FailureTrigger):
    def __init__(self, callType, probability, seed=None):
        self.callType, self.probability = callType, probability
        self.rng = random.Random(seed)

    def triggerFailure(self, callType, iteration, epoch, model):
        return (self.callType in (callType, CallType.ANY)) and self.rng.random() < self.probability


class TimeSinceInitializedTrigger(FailureTrigger):
    def __init__(self, msSinceInit): self.ms, self.t0 = msSinceInit, None
    def initialize(self): self.t0 = time.time()
    def triggerFailure(self, *a): return self.t0 is not None and (time.time() - self.t0) * 1e3 > self.ms


class UserNameTrigger(FailureTrigger):
    def __init__(self, userName): self.userName, self.match = userName, False
    def initialize(self): self.match = getpass.getuser().lower() == self.userName.lower()
    def triggerFailure(self, *a): return self.match


class HostNameTrigger(FailureTrigger):
    def __init__(self, hostName): self.hostName, self.match = hostName, False
    def initialize(self): self.match = socket.gethostname().lower() == self.hostName.lower()
    def triggerFailure(self, *a): return self.match


class IterationEpochTrigger(FailureTrigger):
    def __init__(self, isEpoch, count): self.isEpoch, self.count = isEpoch, count
    def triggerFailure(self, callType, iteration, epoch, model):
        return (epoch == self.count) if self.isEpoch else (iteration == self.count)


class FailureTestingListener(TrainingListener):
    """``FailureTestingListener.java:41-131``: fails the *host* process in a chosen way when a trigger
    fires, to exercise recovery paths (checkpoint reload, process-group timeouts).  Nothing here touches
    the GPU: OOM raises ``MemoryError`` instead of exhausting device memory, the endless sleep is a host
    sleep, exit uses ``os._exit(1)`` between steps."""

    def __init__(self, failureMode, trigger, sleepSeconds=None):
        self.failureMode, self.trigger = failureMode, trigger
        self.sleepSeconds = sleepSeconds           # bound for INFINITE_SLEEP in tests (None = forever)
        self.trigger.initialize()
        self._iter = 0
        self._epoch = 0

    def _call(self, ct, model, iteration=None, epoch=None):
        it = self._iter if iteration is None else iteration
        ep = self._epoch if epoch is None else epoch
        if not self.trigger.triggerFailure(ct, it, ep, model):
            return
        if self.failureMode == FailureMode.OOM:
            raise MemoryError("FailureTestingListener: simulated out-of-memory")
        if self.failureMode == FailureMode.SYSTEM_EXIT_1:
            sys.stdout.flush()
            os._exit(1)
        if self.failureMode == FailureMode.ILLEGAL_STATE:
            raise RuntimeError("FailureTestingListener - generating exception")
        if self.failureMode == FailureMode.INFINITE_SLEEP:
            end = None if self.sleepSeconds is None else time.time() + self.sleepSeconds
            while end is None or time.time() < end:
                time.sleep(0.05 if end is not None else 1.0)
            return
        raise RuntimeError(f"Unknown enum value: {self.failureMode}")

    def iterationDone(self, model, iteration, epoch):
        self._iter, self._epoch = iteration, epoch
        self._call(CallType.ITER_DONE, model, iteration, epoch)

    def onEpochStart(self, model): self._call(CallType.EPOCH_START, model)
    def onEpochEnd(self, model): self._call(CallType.EPOCH_END, model)
    def onForwardPass(self, model, activations=None): self._call(CallType.FORWARD_PASS, model)
    def onGradientCalculation(self, model): self._call(CallType.GRADIENT_CALC, model)
    def onBackwardPass(self, model): self._call(CallType.BACKWARD_PASS, model)
