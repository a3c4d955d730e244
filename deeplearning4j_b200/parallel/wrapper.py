"""``ParallelWrapper`` and ``SharedTrainingMaster``: data-parallel training front ends.

The reference versions (historical API, see ``nd4j/nd4j-common/.../ND4JEnvironmentVars.java:70`` for the
last surviving mention) ran N worker threads in one JVM and exchanged parameters or
threshold-encoded updates through in-process queues / an Aeron mesh.  Here the execution model is
one process per GPU (``torchrun`` or ``launch``): every rank builds the same model, wraps it and
calls ``fit`` on its shard of the data; replicas are kept in sync by the sharing strategy from
``parallel.sharing`` (fused NVLink kernels on B200s, gloo/NCCL collectives otherwise).

``trainingMode``
  * ``AVERAGING`` with ``averagingFrequency == 1``: gradient averaging fused with the updater (one kernel).
  * ``AVERAGING`` with ``averagingFrequency > 1``: local steps, parameters (and optionally updater state)
    averaged every ``f`` iterations — the classic ParallelWrapper behaviour.
  * ``SHARED_GRADIENTS``: threshold-encoded update sharing with residuals.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .sharing import (AdaptiveThresholdAlgorithm, attach_gradient_sharing)


class TrainingMode:
    AVERAGING = "AVERAGING"
    SHARED_GRADIENTS = "SHARED_GRADIENTS"
    CUSTOM = "CUSTOM"


def init_process_group(backend=None):
    """Join the job described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (no-op when single-process)."""
    if dist.is_initialized() or int(os.environ.get("WORLD_SIZE", "1")) <= 1:
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
    if backend == "nccl":
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        dist.init_process_group(backend)


class _ShardedIterator:
    """Rank r of W consumes batches r, r+W, r+2W, ... and stops when any rank would run dry."""

    def __init__(self, base, rank, world):
        self.base, self.rank, self.world = base, rank, world

    def reset(self):
        if hasattr(self.base, "reset"):
            self.base.reset()

    def __iter__(self):
        group = []
        for ds in self.base:
            group.append(ds)
            if len(group) == self.world:
                yield group[self.rank]
                group = []

    def asyncSupported(self):
        return False


class ParallelWrapper:
    def __init__(self, model, workers=None, prefetchBuffer=2, averagingFrequency=1, averageUpdaters=True,
                 reportScoreAfterAveraging=False, trainingMode=TrainingMode.AVERAGING, thresholdAlgorithm=None,
                 residualPostProcessor=None, impl="auto", shardData=True, group=None, workspaceMode=None,
                 gradientsAccumulator=None):
        init_process_group()
        self.model = model
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if workers is not None and workers != self.world and self.world > 1:
            raise ValueError(f"workers({workers}) must equal the number of launched ranks ({self.world})")
        self.prefetchBuffer, self.averagingFrequency = prefetchBuffer, int(averagingFrequency)
        self.averageUpdaters, self.reportScoreAfterAveraging = averageUpdaters, reportScoreAfterAveraging
        self.trainingMode, self.group, self.shardData = trainingMode, group, shardData
        if hasattr(model, "init") and getattr(model, "flat_params", None) is None:
            model.init()
        self.sharing = None
        target = self._target()
        if workspaceMode is not None:
            for setter in ("setTrainingWorkspaceMode", "setInferenceWorkspaceMode"):
                conf = getattr(model, "conf", None)
                if conf is not None and hasattr(conf, setter):
                    getattr(conf, setter)(workspaceMode)
            self.workspaceMode = workspaceMode
        if gradientsAccumulator is not None:
            if trainingMode != TrainingMode.CUSTOM:
                raise ValueError("gradientsAccumulator needs trainingMode(TrainingMode.CUSTOM)")
            target.gradient_hook = gradientsAccumulator
        elif self.world > 1:
            if trainingMode == TrainingMode.SHARED_GRADIENTS:
                self.sharing = attach_gradient_sharing(target, "shared_gradients", impl, thresholdAlgorithm or AdaptiveThresholdAlgorithm(1e-3),
                                                       residualPostProcessor, group)
            elif self.averagingFrequency <= 1:
                self.sharing = attach_gradient_sharing(target, "averaging", impl, group=group)
            else:
                from .sharing import GradientSharing, _Target, _rehome
                from .fused import FusedSharing, SymmetricAllocator, symmetric_available
                self._fused_avg = None
                if impl in ("auto", "fused") and _Target(target).params.is_cuda and symmetric_available():
                    # parameters (and gradients, shadow) move into symmetric memory so that the averaging is one kernel over
                    # peer memory instead of a library all-reduce followed by a divide and a shadow refresh
                    alloc = SymmetricAllocator(group)
                    _rehome(target, alloc)
                    tt = _Target(target)
                    self._fused_avg = FusedSharing(tt.params, tt.grads, tt.shadow, tt.updater, alloc)
                GradientSharing(target, group).broadcast_parameters(0)
                target.gradient_hook = self._param_averaging_hook
        self._local_iter = 0

    def _target(self):
        m = self.model
        if hasattr(m, "trainingConfig"):          # SameDiff
            from ..samediff.training import _ensure_state
            return _ensure_state(m)
        return m

    def _param_averaging_hook(self, target):
        """Classic parameter averaging every ``averagingFrequency`` local steps."""
        from .sharing import _Target
        t = _Target(target)
        it, ep = t.counters()
        t.updater.update(it, ep)
        self._local_iter += 1
        if self._local_iter % self.averagingFrequency == 0:
            if getattr(self, "_fused_avg", None) is not None:
                self._fused_avg.average_parameters()
            else:
                dist.all_reduce(t.params, group=self.group)
                t.params.div_(self.world)
            if self.averageUpdaters and t.updater.state.numel():
                dist.all_reduce(t.updater.state, group=self.group)
                t.updater.state.div_(self.world)
            if getattr(self, "_fused_avg", None) is None:
                t.refresh_shadow()
        if not getattr(t.updater, "_fused_zeroes_grads", False) or not t.params.is_cuda:
            t.grads.zero_()
        return True

    def fit(self, iterator, epochs=1):
        it = _ShardedIterator(iterator, self.rank, self.world) if (self.world > 1 and self.shardData) else iterator
        if hasattr(self.model, "asyncPrefetch"):
            self.model.asyncPrefetch = int(self.prefetchBuffer or 0)   # depth of the model's background batch prefetcher
        self.model.fit(it, epochs)
        if self.reportScoreAfterAveraging and self.world > 1 and hasattr(self.model, "score"):
            s = torch.tensor([float(self.model.score())], dtype=torch.float64, device=self._target().flat_params.device)
            dist.all_reduce(s, group=self.group)
            self.lastAveragedScore = float(s[0]) / self.world
        return self.model

    def shutdown(self):
        t = self._target()
        t.gradient_hook = None

    close = shutdown

    # ------------------------------------------------------------------ builder
    class Builder:
        def __init__(self, model):
            self.model, self.kw = model, {}

        def workers(self, n): self.kw["workers"] = n; return self
        def prefetchBuffer(self, n): self.kw["prefetchBuffer"] = n; return self
        def averagingFrequency(self, n): self.kw["averagingFrequency"] = n; return self
        def averageUpdaters(self, b): self.kw["averageUpdaters"] = b; return self
        def reportScoreAfterAveraging(self, b): self.kw["reportScoreAfterAveraging"] = b; return self
        def trainingMode(self, m): self.kw["trainingMode"] = m; return self
        def thresholdAlgorithm(self, a): self.kw["thresholdAlgorithm"] = a; return self
        def residualPostProcessor(self, p): self.kw["residualPostProcessor"] = p; return self
        def workspaceMode(self, m):
            """Applied to the wrapped model's training/inference workspace mode, as the reference builder does."""
            self.kw["workspaceMode"] = m
            return self

        def gradientsAccumulator(self, a):
            """A custom accumulator object: anything callable as ``hook(target) -> bool`` (TrainingMode.CUSTOM)."""
            if not callable(a):
                raise TypeError("gradientsAccumulator expects a callable gradient hook (target) -> handled?")
            self.kw["gradientsAccumulator"] = a
            return self
        def impl(self, i): self.kw["impl"] = i; return self
        def build(self): return ParallelWrapper(self.model, **self.kw)


class VoidConfiguration:
    """Transport settings of the old parameter-server mesh; only the fields that still mean something here."""

    def __init__(self, unicastPort=40123, networkMask=None, controllerAddress="127.0.0.1", meshBuildMode="MESH"):
        self.unicastPort, self.networkMask, self.controllerAddress, self.meshBuildMode = unicastPort, networkMask, controllerAddress, meshBuildMode

    @staticmethod
    def builder():
        return _KwBuilder(VoidConfiguration)


class _KwBuilder:
    def __init__(self, cls):
        self._cls, self._kw = cls, {}

    def __getattr__(self, k):
        def s(v):
            self._kw[k] = v
            return self
        return s

    def build(self):
        return self._cls(**self._kw)


class SharedTrainingMaster:
    """``SharedTrainingMaster.Builder(voidConfiguration, numWorkers, thresholdAlgorithm, batchSize)``-shaped facade
    over threshold-encoded sharing across ranks (the Spark/Aeron transport is replaced by NVLink peer memory)."""

    def __init__(self, voidConfiguration=None, numWorkers=None, thresholdAlgorithm=None, batchSizePerWorker=32,
                 residualPostProcessor=None, workersPerNode=-1, rddTrainingApproach=None):
        self.voidConfiguration, self.numWorkers = voidConfiguration, numWorkers
        self.thresholdAlgorithm = thresholdAlgorithm or AdaptiveThresholdAlgorithm(1e-3)
        self.batchSizePerWorker, self.residualPostProcessor = batchSizePerWorker, residualPostProcessor

    def wrap(self, model, impl="auto"):
        return ParallelWrapper(model, workers=self.numWorkers, trainingMode=TrainingMode.SHARED_GRADIENTS,
                               thresholdAlgorithm=self.thresholdAlgorithm, residualPostProcessor=self.residualPostProcessor, impl=impl)

    def fit(self, model, iterator, epochs=1):
        return self.wrap(model).fit(iterator, epochs)

    class Builder:
        def __init__(self, *a):
            self.kw = {}
            for v in a:
                if isinstance(v, VoidConfiguration):
                    self.kw["voidConfiguration"] = v
                elif isinstance(v, int) and "numWorkers" not in self.kw:
                    self.kw["numWorkers"] = v
                elif isinstance(v, int):
                    self.kw["batchSizePerWorker"] = v
                elif v is not None:
                    self.kw["thresholdAlgorithm"] = v

        def batchSizePerWorker(self, n): self.kw["batchSizePerWorker"] = n; return self
        def workersPerNode(self, n): self.kw["workersPerNode"] = n; return self
        def thresholdAlgorithm(self, a): self.kw["thresholdAlgorithm"] = a; return self
        def residualPostProcessor(self, p): self.kw["residualPostProcessor"] = p; return self
        def rddTrainingApproach(self, a):
            """Spark RDD export/direct switch: there is no Spark here, only the in-memory ("Direct") behaviour exists."""
            if str(a).rsplit(".", 1)[-1] not in ("Direct", "DIRECT"):
                raise ValueError("only RDDTrainingApproach.Direct is available (no Spark export path in this framework)")
            self.kw["rddTrainingApproach"] = "Direct"
            return self
        def build(self): return SharedTrainingMaster(**self.kw)


def launch(fn, nprocs, *args, backend=None, port=29533):
    """Run ``fn(rank, world, *args)`` in ``nprocs`` processes joined in one process group (CPU: gloo)."""
    import torch.multiprocessing as mp
    mp.spawn(_entry, args=(fn, nprocs, backend, port, args), nprocs=nprocs, join=True)


def _entry(rank, fn, world, backend, port, args):
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank), "MASTER_ADDR": "127.0.0.1",
                       "MASTER_PORT": str(port)})
    init_process_group(backend)
    try:
        fn(rank, world, *args)
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()
