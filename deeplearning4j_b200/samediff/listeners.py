"""SameDiff listeners (``nd4j-api/.../autodiff/listeners``).

Callbacks used by ``SameDiff.fit`` and the sessions: ``epochStart(sd, epoch)``,
``epochEnd(sd, epoch)``, ``iterationDone(sd, iteration, epoch, loss)``, ``preOpExecution(sd, op)``
and ``opExecution(sd, op, outputs)``.  ``ProfilingListener`` writes Chrome trace-event JSON
(``impl/ProfilingListener.java``); on CUDA it brackets every op with events on the current stream
and resolves the durations once at the end, so profiling adds no per-op synchronisation.
"""
from __future__ import annotations

import json
import logging
import os
import threading
import time

import numpy as np
import torch

log = logging.getLogger("deeplearning4j_b200")


class Operation:
    TRAINING = "TRAINING"
    TRAINING_VALIDATION = "TRAINING_VALIDATION"
    INFERENCE = "INFERENCE"
    EVALUATION = "EVALUATION"


class At:
    def __init__(self, epoch=0, iteration=0, trainingThreadNum=0, javaThreadNum=0, frameIter=None, operation=Operation.INFERENCE):
        self.epoch_, self.iteration_, self.operation_ = epoch, iteration, operation

    def epoch(self): return self.epoch_
    def iteration(self): return self.iteration_
    def operation(self): return self.operation_


class Listener:
    def isActive(self, operation): return True
    def epochStart(self, sd, epoch): pass
    def epochEnd(self, sd, epoch): pass
    def iterationStart(self, sd, iteration, epoch, data=None, etlMs=0): pass
    def iterationDone(self, sd, iteration, epoch, loss): pass
    def preOpExecution(self, sd, op): pass
    def opExecution(self, sd, op, outputs): pass
    def operationStart(self, sd, operation): pass
    def operationEnd(self, sd, operation): pass


BaseListener = Listener


class ScoreListener(Listener):
    """``impl/ScoreListener.java:105,149``: loss (and batches/sec, samples/sec) every ``frequency`` iterations."""

    def __init__(self, frequency=10, reportEpochs=True, reportIterPerformance=True, out=None):
        self.frequency, self.reportEpochs, self.reportIterPerformance = max(int(frequency), 1), reportEpochs, reportIterPerformance
        self.out = out
        self._t = None
        self._n = 0
        self.messages = []

    def _emit(self, msg):
        self.messages.append(msg)
        log.info(msg) if self.out is None else print(msg, file=self.out)

    def epochStart(self, sd, epoch):
        if self.reportEpochs:
            self._emit(f"Starting epoch {epoch}")
        self._t, self._n = time.perf_counter(), 0

    def iterationDone(self, sd, iteration, epoch, loss):
        self._n += 1
        if iteration % self.frequency:
            return
        val = float(loss)
        msg = f"Loss at epoch {epoch}, iteration {iteration}: {val:.6g}"
        if self.reportIterPerformance and self._t is not None:
            dt = max(time.perf_counter() - self._t, 1e-9)
            msg += f" ({self._n / dt:.2f} batches/sec)"
            self._t, self._n = time.perf_counter(), 0
        self._emit(msg)

    def epochEnd(self, sd, epoch):
        if self.reportEpochs:
            self._emit(f"Finished epoch {epoch}")


class HistoryListener(Listener):
    """Collects per-iteration losses and epoch times (``impl/HistoryListener.java``)."""

    def __init__(self, trainingConfig=None):
        self.losses, self.epochTimes, self._t = [], [], None

    def epochStart(self, sd, epoch):
        self._t = time.perf_counter()
        self.losses.append([])

    def iterationDone(self, sd, iteration, epoch, loss):
        if not self.losses:
            self.losses.append([])
        self.losses[-1].append(loss)

    def epochEnd(self, sd, epoch):
        self.epochTimes.append(time.perf_counter() - (self._t or time.perf_counter()))

    def getReport(self):
        return {"lossCurve": [[float(l) for l in e] for e in self.losses], "epochTimes": list(self.epochTimes)}


class CheckpointListener(Listener):
    """``impl/checkpoint/CheckpointListener.java``: saves ``checkpoint-<n>.sdnb`` style files on an
    iteration / epoch / time schedule with keep-all or keep-last retention and a ``checkpointInfo.txt`` index."""

    def __init__(self, rootDir, saveEveryNIterations=None, saveEveryNEpochs=None, saveEveryMs=None, keepLast=0, keepEvery=0,
                 saveUpdaterState=True, fileFormat="fb", deleteExisting=False):
        self.rootDir = str(rootDir)
        os.makedirs(self.rootDir, exist_ok=True)
        if deleteExisting:
            for f in os.listdir(self.rootDir):
                if f.startswith("checkpoint-") or f == "checkpointInfo.txt":
                    os.remove(os.path.join(self.rootDir, f))
        self.saveEveryNIterations, self.saveEveryNEpochs, self.saveEveryMs = saveEveryNIterations, saveEveryNEpochs, saveEveryMs
        self.keepLast, self.keepEvery, self.saveUpdaterState, self.fileFormat = keepLast, keepEvery, saveUpdaterState, fileFormat
        self.checkpoints = []
        self._num = -1
        self._last = time.time()

    class Builder:
        def __init__(self, rootDir): self.kw = {"rootDir": rootDir}
        def saveEveryNIterations(self, n): self.kw["saveEveryNIterations"] = n; return self
        def saveEveryNEpochs(self, n): self.kw["saveEveryNEpochs"] = n; return self
        saveEveryEpoch = lambda self: self.saveEveryNEpochs(1)
        def saveEvery(self, amount_ms): self.kw["saveEveryMs"] = amount_ms; return self
        def keepAll(self): self.kw["keepLast"] = 0; return self
        def keepLast(self, n): self.kw["keepLast"] = n; return self
        def keepLastAndEvery(self, n, e): self.kw["keepLast"], self.kw["keepEvery"] = n, e; return self
        def saveUpdaterState(self, b): self.kw["saveUpdaterState"] = b; return self
        def deleteExisting(self, b): self.kw["deleteExisting"] = b; return self
        def build(self): return CheckpointListener(**self.kw)

    @staticmethod
    def builder(rootDir): return CheckpointListener.Builder(rootDir)

    def iterationDone(self, sd, iteration, epoch, loss):
        if self.saveEveryNIterations and iteration > 0 and iteration % self.saveEveryNIterations == 0:
            self._save(sd, iteration, epoch)
        elif self.saveEveryMs and (time.time() - self._last) * 1e3 >= self.saveEveryMs:
            self._save(sd, iteration, epoch)

    def epochEnd(self, sd, epoch):
        if self.saveEveryNEpochs and (epoch + 1) % self.saveEveryNEpochs == 0:
            self._save(sd, sd.trainingConfig.iterationCount, epoch)

    def _save(self, sd, iteration, epoch):
        self._num += 1
        fn = f"checkpoint-{self._num}_epoch-{epoch}_iter-{iteration}.{'sdnb' if self.fileFormat == 'sdnb' else 'bin'}"
        path = os.path.join(self.rootDir, fn)
        if self.fileFormat == "sdnb":
            sd.save(path, self.saveUpdaterState)
        else:
            sd.asFlatFile(path, self.saveUpdaterState)
        rec = os.path.join(self.rootDir, "checkpointInfo.txt")
        new = not os.path.exists(rec)
        with open(rec, "a") as f:
            if new:
                f.write("checkpointNum,timestamp,iteration,epoch,filename\n")
            f.write(f"{self._num},{int(time.time() * 1e3)},{iteration},{epoch},{fn}\n")
        self.checkpoints.append((self._num, fn))
        self._last = time.time()
        if self.keepLast:
            keep = {n for n, _ in self.checkpoints[-self.keepLast:]}
            for n, f in list(self.checkpoints):
                if n in keep or (self.keepEvery and n % self.keepEvery == 0):
                    continue
                p = os.path.join(self.rootDir, f)
                if os.path.exists(p):
                    os.remove(p)
                self.checkpoints.remove((n, f))

    def availableCheckpoints(self):
        return [(n, os.path.join(self.rootDir, f)) for n, f in self.checkpoints]

    def loadLast(self, loadUpdaterState=True):
        from .core import SameDiff
        if not self.checkpoints:
            return None
        p = os.path.join(self.rootDir, self.checkpoints[-1][1])
        return SameDiff.load(p, loadUpdaterState) if p.endswith(".sdnb") else SameDiff.fromFlatFile(p, loadUpdaterState)


class ProfilingListener(Listener):
    """Chrome trace-event profile of op execution (load the output in chrome://tracing or Perfetto)."""

    def __init__(self, outputFile, all=True, warmup=0, nIter=-1, nMs=-1, operations=None):
        self.outputFile, self.warmup, self.nIter, self.nMs = str(outputFile), warmup, nIter, nMs
        self.operations = operations
        self.events = []
        self._pending = []          # (name, op, start_evt, end_evt, host_ts, tid)
        self._open = {}
        self._iters = 0
        self._t0 = time.perf_counter()
        self._closed = False

    class Builder:
        def __init__(self, f): self.kw = {"outputFile": f}
        def recordAll(self): return self
        def warmup(self, n): self.kw["warmup"] = n; return self
        def maxProfileIterations(self, n): self.kw["nIter"] = n; return self
        def maxProfilerMilliseconds(self, ms): self.kw["nMs"] = ms; return self
        def operations(self, *ops): self.kw["operations"] = list(ops); return self
        def build(self): return ProfilingListener(**self.kw)

    @staticmethod
    def builder(f): return ProfilingListener.Builder(f)

    def _active(self):
        if self._closed or self._iters < self.warmup:
            return False
        if self.nIter > 0 and self._iters >= self.warmup + self.nIter:
            return False
        if self.nMs > 0 and (time.perf_counter() - self._t0) * 1e3 > self.nMs:
            return False
        return True

    def preOpExecution(self, sd, op):
        if not self._active():
            return
        cuda = sd.device.type == "cuda"
        ev = None
        if cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            if getattr(self, "nvtx", True):
                torch.cuda.nvtx.range_push(f"{op.opName}:{op.name}")        # named range per op for external profilers
        self._open[id(op)] = (ev, time.perf_counter())

    def opExecution(self, sd, op, outputs):
        st = self._open.pop(id(op), None)
        if st is None:
            return
        ev0, t_host = st
        if ev0 is not None and getattr(self, "nvtx", True):
            torch.cuda.nvtx.range_pop()
        shapes = [list(o.shape) for o in outputs if isinstance(o, torch.Tensor)]
        args = {"op": op.opName, "inputs": [i for i in op.inputs if i is not None], "outputs": list(op.outputs), "output shapes": shapes}
        if ev0 is not None:
            ev1 = torch.cuda.Event(enable_timing=True)
            ev1.record()
            self._pending.append((op.name, args, ev0, ev1, t_host))
        else:
            dur = time.perf_counter() - t_host
            self.events.append({"name": op.name, "cat": "op", "ph": "X", "ts": int((t_host - self._t0) * 1e6), "dur": max(int(dur * 1e6), 1),
                                "pid": os.getpid(), "tid": threading.get_ident() % 100000, "args": args})

    def iterationDone(self, sd, iteration, epoch, loss):
        self._iters += 1
        if self.nIter > 0 and self._iters >= self.warmup + self.nIter and not self._closed:
            self.close()

    def operationEnd(self, sd, operation):
        self.close()

    def _resolve(self):
        if not self._pending:
            return
        torch.cuda.synchronize()
        base_ev, base_host = self._pending[0][2], self._pending[0][4]
        for name, args, e0, e1, t_host in self._pending:
            ts = (base_host - self._t0) * 1e6 + base_ev.elapsed_time(e0) * 1e3
            self.events.append({"name": name, "cat": "op", "ph": "X", "ts": int(ts), "dur": max(int(e0.elapsed_time(e1) * 1e3), 1),
                                "pid": os.getpid(), "tid": 0, "args": args})
        self._pending = []

    def close(self):
        self._resolve()
        with open(self.outputFile, "w") as f:
            json.dump({"traceEvents": self.events, "displayTimeUnit": "ms"}, f)
        self._closed = True


class OpBenchmarkListener(Listener):
    """Aggregated time per op name (``impl/OpBenchmarkListener.java``).  On CUDA every op is bracketed by
    events and durations are resolved in ``getAggregateModeMap`` / ``printTimings``."""

    def __init__(self, operation=Operation.INFERENCE, mode="AGGREGATE", minRuntime=0):
        self.mode, self.minRuntime = mode, minRuntime
        self._open, self._pending, self.timings = {}, [], {}

    def preOpExecution(self, sd, op):
        if sd.device.type == "cuda":
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._open[id(op)] = e
        else:
            self._open[id(op)] = time.perf_counter()

    def opExecution(self, sd, op, outputs):
        st = self._open.pop(id(op), None)
        if st is None:
            return
        if isinstance(st, float):
            self._add(op, (time.perf_counter() - st) * 1e3)
        else:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._pending.append((op, st, e))

    def _add(self, op, ms):
        key = op.opName if self.mode == "AGGREGATE" else op.name
        t = self.timings.setdefault(key, {"count": 0, "totalMs": 0.0, "opName": op.opName})
        t["count"] += 1
        t["totalMs"] += ms

    def getAggregateModeMap(self):
        if self._pending:
            torch.cuda.synchronize()
            for op, a, b in self._pending:
                self._add(op, a.elapsed_time(b))
            self._pending = []
        return self.timings

    def printTimings(self):
        rows = sorted(self.getAggregateModeMap().items(), key=lambda kv: -kv[1]["totalMs"])
        return "\n".join(f"{k:<40}{v['count']:>8}{v['totalMs']:>12.3f} ms{v['totalMs'] / v['count']:>12.4f} ms/call" for k, v in rows)


class ExecDebuggingListener(Listener):
    """Prints each op as it executes (``impl/ExecDebuggingListener.java``): OPS_ONLY, SHAPES_ONLY or REPRODUCE."""

    def __init__(self, printMode="OPS_ONLY", maxIterations=-1, logIter=False, out=None):
        self.printMode, self.maxIterations, self.logIter, self.out = printMode, maxIterations, logIter, out
        self._count, self._step = 0, 0
        self.lines = []

    def opExecution(self, sd, op, outputs):
        if 0 < self.maxIterations <= self._count:
            return
        line = f"(iter={self._count},op={self._step}) {op.name} ({op.opName}) inputs={op.inputs} -> {op.outputs}"
        if self.printMode != "OPS_ONLY":
            line += " shapes=" + str([tuple(o.shape) for o in outputs if isinstance(o, torch.Tensor)])
        if self.printMode == "REPRODUCE":
            line += f" args={ {k: v for k, v in op.args.items() if not callable(v)} }"
        self._step += 1
        self.lines.append(line)
        log.info(line) if self.out is None else print(line, file=self.out)

    def iterationDone(self, sd, iteration, epoch, loss):
        self._count += 1
        self._step = 0


class ArraySavingListener(Listener):
    """Saves every op output as ``<dir>/<iteration>_<n>_<name>.npy`` (``debugging/ArraySavingListener.java``)."""

    def __init__(self, directory):
        self.dir = str(directory)
        os.makedirs(self.dir, exist_ok=True)
        self._iter, self._n = 0, 0

    def opExecution(self, sd, op, outputs):
        for name, o in zip(op.outputs, outputs):
            if isinstance(o, torch.Tensor):
                arr = o.detach().float().cpu().numpy() if o.dtype == torch.bfloat16 else o.detach().cpu().numpy()
                np.save(os.path.join(self.dir, f"{self._iter}_{self._n}_{name.replace('/', '__').replace(':', '_')}.npy"), arr)
                self._n += 1

    def iterationDone(self, sd, iteration, epoch, loss):
        self._iter += 1
        self._n = 0

    @staticmethod
    def compare(dir1, dir2, eps=1e-5):
        bad = []
        for f in sorted(os.listdir(dir1)):
            p2 = os.path.join(dir2, f)
            if not os.path.exists(p2):
                bad.append((f, "missing"))
                continue
            a, b = np.load(os.path.join(dir1, f)), np.load(p2)
            if a.shape != b.shape or not np.allclose(a, b, atol=eps, rtol=eps, equal_nan=True):
                bad.append((f, "differs"))
        return bad


class UIListener(Listener):
    """Writes graph structure and training events as JSON lines that ``ui.server`` can serve
    (the reference writes ``uigraphevents.fbs`` / ``uigraphstatic.fbs`` records to a log file)."""

    def __init__(self, logFile, lossFrequency=1, updateRatioFrequency=0, fileMode="CREATE_OR_APPEND"):
        self.logFile, self.lossFrequency = str(logFile), max(int(lossFrequency), 1)
        if fileMode == "CREATE_APPEND_NOCHECK" or not os.path.exists(self.logFile):
            open(self.logFile, "a").close()
        self._wrote_graph = False

    def _write(self, rec):
        with open(self.logFile, "a") as f:
            f.write(json.dumps(rec) + "\n")

    def epochStart(self, sd, epoch):
        if not self._wrote_graph:
            self._write({"type": "graph", "variables": [{"name": n, "type": v.variableType, "dtype": getattr(v._dtype, "name", None),
                                                          "shape": list(v._shape) if v._shape else None} for n, v in sd.variables.items()],
                         "ops": [{"name": o.name, "op": o.opName, "inputs": o.inputs, "outputs": o.outputs} for o in sd.ops]})
            self._wrote_graph = True
        self._write({"type": "epochStart", "epoch": epoch, "time": time.time()})

    def iterationDone(self, sd, iteration, epoch, loss):
        if iteration % self.lossFrequency == 0:
            self._write({"type": "loss", "iteration": iteration, "epoch": epoch, "loss": float(loss), "time": time.time()})

    def epochEnd(self, sd, epoch):
        self._write({"type": "epochEnd", "epoch": epoch, "time": time.time()})
