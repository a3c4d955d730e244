"""Op profiling and NaN/Inf panics (``nd4j-api/.../linalg/profiler``: ``OpProfiler``, ``ProfilerConfig``;
``OpExecutioner.ProfilingMode`` ``api/ops/executioner/OpExecutioner.java:50``).

``OpExecutioner`` is the eager entry point ``exec(opName, inputs, **args)`` over the op registry; with a
profiling mode set it times every op (CUDA events when the inputs live on a GPU, resolved lazily) and can
check outputs for NaN / Inf like the reference's NAN_PANIC / INF_PANIC / ANY_PANIC modes."""
from __future__ import annotations

import time
from dataclasses import dataclass

import torch

from ..nd.ndarray import INDArray
from ..ops import registry


class ProfilingMode:
    DISABLED = "DISABLED"
    NAN_PANIC = "NAN_PANIC"
    INF_PANIC = "INF_PANIC"
    ANY_PANIC = "ANY_PANIC"
    OPERATIONS = "OPERATIONS"
    METHODS = "METHODS"
    ALL = "ALL"
    SCOPE_PANIC = "SCOPE_PANIC"
    BANDWIDTH = "BANDWIDTH"


@dataclass
class ProfilerConfig:
    checkForNAN: bool = False
    checkForINF: bool = False
    stackTrace: bool = False
    checkElapsedTime: bool = False
    checkWorkspaces: bool = False
    checkLocality: bool = False
    checkBandwidth: bool = False
    nativeStatistics: bool = False

    @staticmethod
    def builder():
        class B:
            def __init__(s): s.kw = {}
            def __getattr__(s, k):
                if k.startswith("_") or k == "kw":
                    raise AttributeError(k)
                def f(v=True):
                    s.kw[k] = v
                    return s
                return f
            def build(s): return ProfilerConfig(**s.kw)
        return B()


class ND4JOpProfilerException(RuntimeError):
    pass


class OpProfiler:
    _instance = None

    def __init__(self):
        self.config = ProfilerConfig()
        self.reset()

    @classmethod
    def getInstance(cls):
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def reset(self):
        self.invocations = 0
        self.op_counter = {}
        self.op_time_ms = {}
        self.class_counter = {}
        self._pending = []
        self.bytes_moved = {}

    def setConfig(self, c): self.config = c
    def getConfig(self): return self.config
    def getInvocationsCount(self): return self.invocations

    def processOpCall(self, name, group=""):
        self.invocations += 1
        self.op_counter[name] = self.op_counter.get(name, 0) + 1
        if group:
            self.class_counter[group] = self.class_counter.get(group, 0) + 1

    def timeOpCall(self, name, ms):
        self.op_time_ms[name] = self.op_time_ms.get(name, 0.0) + ms

    def _defer(self, name, e0, e1): self._pending.append((name, e0, e1))

    def _resolve(self):
        if self._pending:
            torch.cuda.synchronize()
            for n, a, b in self._pending:
                self.timeOpCall(n, a.elapsed_time(b))
            self._pending = []

    def getStatistics(self):
        self._resolve()
        return {"invocations": self.invocations, "opCounter": dict(self.op_counter), "opTimeMs": dict(self.op_time_ms),
                "classCounter": dict(self.class_counter)}

    def printOutDashboard(self):
        st = self.getStatistics()
        lines = ["---Total Op Calls: %d" % st["invocations"], "", "Top ops by time:"]
        for n, ms in sorted(st["opTimeMs"].items(), key=lambda kv: -kv[1])[:25]:
            c = st["opCounter"].get(n, 0)
            lines.append(f"  {n:<40}{c:>8} calls {ms:>12.3f} ms {ms / max(c, 1):>10.4f} ms/call")
        return "\n".join(lines)

    @staticmethod
    def checkForNaN(name, outs):
        for o in outs:
            if isinstance(o, torch.Tensor) and o.is_floating_point() and bool(torch.isnan(o).any()):
                raise ND4JOpProfilerException(f"P.A.N.I.C.! Op.Z() contains NaN value(s): op {name}")

    @staticmethod
    def checkForInf(name, outs):
        for o in outs:
            if isinstance(o, torch.Tensor) and o.is_floating_point() and bool(torch.isinf(o).any()):
                raise ND4JOpProfilerException(f"P.A.N.I.C.! Op.Z() contains Inf value(s): op {name}")


class OpExecutioner:
    """Eager op execution over the registry (``Nd4j.getExecutioner().exec(op)``)."""
    _instance = None

    def __init__(self):
        self.profilingMode = ProfilingMode.DISABLED
        self.profiler = OpProfiler.getInstance()

    @classmethod
    def getInstance(cls):
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def setProfilingMode(self, mode): self.profilingMode = mode
    def getProfilingMode(self): return self.profilingMode

    def setProfilingConfig(self, config):
        self.profiler.setConfig(config)
        if config.checkForNAN and config.checkForINF:
            self.profilingMode = ProfilingMode.ANY_PANIC
        elif config.checkForNAN:
            self.profilingMode = ProfilingMode.NAN_PANIC
        elif config.checkForINF:
            self.profilingMode = ProfilingMode.INF_PANIC
        elif config.checkElapsedTime:
            self.profilingMode = ProfilingMode.OPERATIONS

    def exec(self, opName, inputs=(), **args):
        d = registry.get(opName)
        ins = [i.t if isinstance(i, INDArray) else i for i in inputs]
        mode = self.profilingMode
        timing = mode in (ProfilingMode.OPERATIONS, ProfilingMode.ALL, ProfilingMode.METHODS)
        cuda = timing and any(isinstance(i, torch.Tensor) and i.is_cuda for i in ins)
        if timing:
            if cuda:
                e0 = torch.cuda.Event(enable_timing=True)
                e0.record()
            else:
                t0 = time.perf_counter()
        out = d.fn(*ins, **args)
        outs = list(out) if isinstance(out, (tuple, list)) else [out]
        if mode != ProfilingMode.DISABLED:
            self.profiler.processOpCall(opName, d.group)
            if timing:
                if cuda:
                    e1 = torch.cuda.Event(enable_timing=True)
                    e1.record()
                    self.profiler._defer(opName, e0, e1)
                else:
                    self.profiler.timeOpCall(opName, (time.perf_counter() - t0) * 1e3)
            if mode in (ProfilingMode.NAN_PANIC, ProfilingMode.ANY_PANIC):
                OpProfiler.checkForNaN(opName, outs)
            if mode in (ProfilingMode.INF_PANIC, ProfilingMode.ANY_PANIC):
                OpProfiler.checkForInf(opName, outs)
        wrap = lambda o: INDArray(o) if isinstance(o, torch.Tensor) else o
        return [wrap(o) for o in outs] if isinstance(out, (tuple, list)) else wrap(out)

    def execAndReturn(self, opName, inputs=(), **args): return self.exec(opName, inputs, **args)

    def commit(self):
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def getEnvironmentInformation(self):
        from .environment import Environment
        return Environment.getInstance().describe()

    def printEnvironmentInformation(self):
        for k, v in self.getEnvironmentInformation().items():
            print(f"{k}: {v}")
