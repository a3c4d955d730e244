"""Machinery shared by ``MultiLayerNetwork`` and ``ComputationGraph``: the flattened
parameter / gradient buffers and their per-layer views, parameter initialisation, the
updater, listeners, score bookkeeping and the training-step skeleton.

Parity: ``nn/multilayer/MultiLayerNetwork.java:604-800`` (``init``: one flat parameter array,
layers get views; ``flattenedGradients`` ``:789-800``), ``optimize/solvers/
StochasticGradientDescent.java:49-78`` (gradient -> updater -> step -> listeners).
"""
from __future__ import annotations

import time

import numpy as np
import torch

from ..nd.dtype import DataType
from ..nd.ndarray import INDArray, wrap, _unwrap
from .conf.base import ParamSpec, flat_view
from .updater import MultiLayerUpdater, ParamEntry
from ..utils import nvtx as _nvtx


def _as_tensor(x, device=None, dtype=None):
    if x is None:
        return None
    t = _unwrap(x)
    if not isinstance(t, torch.Tensor):
        t = torch.as_tensor(np.asarray(t))
    if device is not None and t.device != device:
        t = t.to(device, non_blocking=True)
    if dtype is not None and t.dtype != dtype and t.dtype.is_floating_point:
        t = t.to(dtype)
    return t


class BaseNetwork:
    def __init__(self):
        self.flat_params = None
        self.flat_grads = None
        self.entries: list = []
        self.param_views: dict = {}     # owner key -> {name: leaf tensor (requires grad)}
        self.updater: MultiLayerUpdater | None = None
        self.listeners: list = []
        self._score = None
        self._last_batch = 0
        self.iterationCount = 0
        self.epochCount = 0
        self.device = torch.device("cpu")
        self._last_etl_ms = 0.0
        self.gradient_hook = None       # set by ParallelWrapper: called between backward and the updater
        self.flat_shadow = None
        self.shadow_offsets = None
        self.asyncPrefetch = 2          # depth of the background batch prefetcher used by fit(iterator)

    # ------------------------------------------------------------------ to be provided by subclasses
    def _owners(self):
        """Ordered list of (key, layer) with parameters, in flattening order."""
        raise NotImplementedError

    def _param_dtype(self) -> torch.dtype:
        return self.conf.dataType.to_torch()

    def _compute_dtype(self) -> torch.dtype:
        cd = getattr(self.conf, "computeDataType", None)
        return cd.to_torch() if cd is not None else self._param_dtype()

    # ------------------------------------------------------------------ init
    def _init_params(self, params=None, clone=True, seed=0):
        owners = self._owners()
        entries, off = [], 0
        for idx, (key, layer) in enumerate(owners):
            for spec in layer.param_specs():
                entries.append(ParamEntry(idx, layer, spec, off, f"{key}_{spec.name}"))
                off += spec.numel
        self.entries = entries
        n = off
        dt = self._param_dtype()
        if params is not None:
            p = _as_tensor(params).reshape(-1)
            if p.numel() != n:
                raise ValueError(f"Invalid parameters: expected length {n}, got {p.numel()}")
            p = p.to(dt).to(self.device)
            self.flat_params = p.clone() if clone else p
        else:
            self.flat_params = torch.zeros(n, dtype=dt, device=self.device)
            gen = torch.Generator(device=self.device)
            gen.manual_seed(int(seed))
            with torch.no_grad():
                for e in entries:
                    self._init_one(e, gen)
        self.flat_grads = torch.zeros(n, dtype=dt, device=self.device)
        self._make_views()

    def _init_one(self, e: ParamEntry, gen):
        spec, layer = e.spec, e.layer
        seg = self.flat_params[e.offset:e.end]
        view = flat_view(self.flat_params, e.offset, spec)
        init = spec.init
        if callable(init):
            init(view, gen)
        elif isinstance(init, (int, float)) and not isinstance(init, bool):
            seg.fill_(float(init))
        elif spec.kind == "bias":
            seg.fill_(float(getattr(layer, "biasInit", 0.0) or 0.0))
        elif spec.kind == "gain":
            seg.fill_(float(getattr(layer, "gainInit", 1.0) or 1.0))
        elif spec.kind == "state":
            seg.zero_()
        else:
            wi = getattr(layer, "weightInit", None)
            if init == "recurrent" and getattr(layer, "weightInitRecurrent", None) is not None:
                wi = layer.weightInitRecurrent
            if wi is None:
                from .weights import WeightInit
                wi = WeightInit.get("XAVIER")
            # draw into a contiguous scratch in logical order, then store through the view
            tmp = torch.empty(spec.shape, dtype=torch.float32, device=self.device)
            wi.init(spec.fanIn, spec.fanOut, tmp, gen)
            view.copy_(tmp.to(view.dtype))

    def _make_views(self):
        self.param_views = {}
        owners = self._owners()
        self._make_shadow()
        for i, e in enumerate(self.entries):
            key = owners[e.layer_index][0]
            v = flat_view(self.flat_params, e.offset, e.spec).detach()
            if e.spec.kind != "state":
                v.requires_grad_(True)
                v.grad = flat_view(self.flat_grads, e.offset, e.spec)
                if self.flat_shadow is not None:
                    v._lp = flat_view(self.flat_shadow, self.shadow_offsets[i], e.spec)
            self.param_views.setdefault(key, {})[e.spec.name] = v

    def _make_shadow(self):
        """Low-precision copy of the parameters for the tensor-core GEMMs (fp32 master weights stay
        in ``flat_params``).  Every parameter starts on a 16-byte boundary so TMA can address it."""
        self.flat_shadow, self.shadow_offsets = None, None
        cd = self._compute_dtype()
        if cd == self._param_dtype() or self.flat_params is None or not self.flat_params.is_cuda:
            return
        offs, off = [], 0
        for e in self.entries:
            offs.append(off)
            off += (e.spec.numel + 63) // 64 * 64
        self.shadow_offsets = offs
        alloc = getattr(self, "_flat_allocator", None)
        self.flat_shadow = alloc(off, cd, self.device) if alloc is not None else torch.zeros(max(off, 1), dtype=cd, device=self.device)
        self._refresh_shadow()

    def _refresh_shadow(self):
        if self.flat_shadow is None:
            return
        with torch.no_grad():
            for e, so in zip(self.entries, self.shadow_offsets):
                self.flat_shadow[so:so + e.spec.numel].copy_(self.flat_params[e.offset:e.end])

    def _rebind(self):
        """Call after the flat buffers were replaced (device move, setParams with new storage)."""
        self._make_views()
        if self.updater is not None:
            self.updater.params, self.updater.grads = self.flat_params, self.flat_grads
            self.updater.shadow, self.updater.shadow_offsets = self.flat_shadow, self.shadow_offsets
            self.updater._native_tables = None
        # graphs captured earlier read the old parameter / shadow storage and write the old gradient buffer
        cg = getattr(self, "_cg", None)
        if cg is not None:
            cg["entries"] = {}

    def _ensure_updater(self):
        if self.updater is None:
            self.updater = MultiLayerUpdater(self.entries, self.flat_params, self.flat_grads)
        self.updater.shadow, self.updater.shadow_offsets = self.flat_shadow, self.shadow_offsets
        return self.updater

    # ------------------------------------------------------------------ device
    def to(self, device):
        device = torch.device(device)
        if device == self.device:
            return self
        self.device = device
        self.flat_params = self.flat_params.to(device)
        self.flat_grads = self.flat_grads.to(device)
        if self.updater is not None:
            self.updater.state = self.updater.state.to(device)
            self.updater._bind()
        self._rebind()
        return self

    def cuda(self, idx=0):
        return self.to(f"cuda:{idx}")

    # ------------------------------------------------------------------ params API
    def params(self):
        return INDArray(self.flat_params)

    def numParams(self):
        return int(self.flat_params.numel())

    def setParams(self, p):
        t = _as_tensor(p).reshape(-1)
        with torch.no_grad():
            self.flat_params.copy_(t.to(self.flat_params.dtype).to(self.device))
        self._refresh_shadow()

    setParameters = setParams

    def gradient(self):
        from .gradient import Gradient
        return Gradient(self)

    def getFlattenedGradients(self):
        return INDArray(self.flat_grads)

    def paramTable(self):
        owners = self._owners()
        out = {}
        for e in self.entries:
            key = owners[e.layer_index][0]
            out[f"{key}_{e.spec.name}"] = INDArray(flat_view(self.flat_params, e.offset, e.spec))
        return out

    def getParam(self, key):
        return self.paramTable()[key]

    def setParam(self, key, value):
        with torch.no_grad():
            self.paramTable()[key].t.copy_(_as_tensor(value).to(self.device))

    def getUpdater(self):
        return self._ensure_updater()

    def setUpdater(self, u):
        self.updater = u

    # ------------------------------------------------------------------ listeners
    def setListeners(self, *ls):
        if len(ls) == 1 and isinstance(ls[0], (list, tuple)):
            ls = ls[0]
        self.listeners = list(ls)

    def addListeners(self, *ls):
        self.listeners.extend(ls)

    def getListeners(self):
        return self.listeners

    def _fire(self, name, *a):
        for l in self.listeners:
            fn = getattr(l, name, None)
            if fn is not None:
                fn(self, *a)

    # ------------------------------------------------------------------ score
    def score(self, *a):
        if a:
            return self._score_dataset(*a)
        s = self._score
        if s is None:
            return 0.0
        return float(s)

    def setScore(self, s):
        self._score = s

    def _regularization_score(self):
        tot = None
        for e in self.entries:
            if e.spec.kind == "state":
                continue
            regs = e.layer.regularizers(e.spec)
            if not regs:
                continue
            p = self.flat_params[e.offset:e.end]
            for r in regs:
                v = r.score(p, self.iterationCount, self.epochCount)
                tot = v if tot is None else tot + v
        return tot

    def getIterationCount(self): return self.iterationCount
    def getEpochCount(self): return self.epochCount
    def setIterationCount(self, i): self.iterationCount = int(i); self.conf.iterationCount = int(i)
    def setEpochCount(self, e): self.epochCount = int(e); self.conf.epochCount = int(e)
    def incrementEpochCount(self): self.setEpochCount(self.epochCount + 1)
    def batchSize(self): return self._last_batch
    def getLastEtlTime(self): return self._last_etl_ms
    def setLastEtlTime(self, ms): self._last_etl_ms = ms

    # ------------------------------------------------------------------ CUDA-graph capture of forward + backward
    def setCudaGraphs(self, enabled=True, warmup=1):
        """Capture the loss + backward pass of a training step into a CUDA graph (one per input signature) and replay it
        on later steps, which removes the per-kernel launch cost of launch-bound networks.  The first ``warmup`` steps
        of a signature run eagerly; the updater / gradient-sharing step stays outside the graph so schedules and
        iteration-dependent hyper-parameters keep working.  Steps with masks or carried recurrent state run eagerly."""
        self._cg = {"on": bool(enabled), "warmup": int(warmup), "entries": {}}
        return self

    def _loss_backward(self, tensors, loss_fn, eager_ok=True, aux=None):
        """Runs ``loss = loss_fn(tensors); loss.backward()`` either eagerly or through a captured CUDA graph.
        ``tensors`` is a flat list of input / label (/ carried state) tensors; returns the detached loss.  ``aux`` is a
        dict that ``loss_fn`` fills with side outputs (carried recurrent state); on replay it receives the captured
        graph's output tensors."""
        cg = getattr(self, "_cg", None)
        if not (cg and cg["on"] and eager_ok and self.flat_params.is_cuda):
            loss = loss_fn(tensors)
            loss.backward()
            return loss.detach()
        from ..ops import native
        key = tuple((tuple(t.shape), t.dtype, tuple(t.stride())) for t in tensors)
        e = cg["entries"].setdefault(key, {"seen": 0, "graph": None})
        if e["graph"] is None:
            e["seen"] += 1
            if e["seen"] <= cg["warmup"]:
                loss = loss_fn(tensors)
                loss.backward()
                return loss.detach()
            e["static"] = [t.clone() for t in tensors]
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            n0 = native.LAUNCHES
            with torch.cuda.graph(g):
                loss = loss_fn(e["static"])
                loss.backward()
            e["launches"] = native.LAUNCHES - n0
            native.LAUNCHES = n0                    # capture launched nothing
            e["loss"] = loss.detach()
            e["aux"] = dict(aux) if aux is not None else None
            e["graph"] = g
        for dst, src in zip(e["static"], tensors):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src, non_blocking=True)
        e["graph"].replay()
        native.LAUNCHES += e["launches"]
        if aux is not None and e["aux"] is not None:
            aux.clear()
            aux.update(e["aux"])
        return e["loss"]

    # ------------------------------------------------------------------ step skeleton
    def _apply_update(self):
        with _nvtx.range("updater"):
            return self._apply_update_impl()

    def _apply_update_impl(self):
        """updater -> step (-> constraints), between backward and ``iterationDone``."""
        if self.gradient_hook is not None:
            if self.gradient_hook(self) is True:   # hook consumed the gradient and stepped the params
                return
        upd = self._ensure_updater()
        upd.shadow, upd.shadow_offsets = self.flat_shadow, self.shadow_offsets
        upd.update(self.iterationCount, self.epochCount)
        if self.flat_shadow is not None and not getattr(upd, "_shadow_fresh", False):
            self._refresh_shadow()
        self._apply_constraints()

    def _apply_constraints(self):
        for e in self.entries:
            cs = getattr(e.layer, "constraints", None)
            if cs and e.spec.kind in ("weight",):
                with torch.no_grad():
                    v = flat_view(self.flat_params, e.offset, e.spec)
                    for c in cs:
                        if c.params is None or e.spec.name in c.params:
                            c.apply(v)

    def _iteration_done(self):
        self.iterationCount += 1
        self.conf.iterationCount = self.iterationCount
        if self.listeners:
            self._fire("iterationDone", self.iterationCount - 1, self.epochCount)

    def clearGradients(self):
        self.flat_grads.zero_()

    # ------------------------------------------------------------------ fit over iterators
    def _fit_iterator(self, it, epochs=1):
        from ..data.iterators import AsyncDataSetIterator
        for _ in range(epochs):
            if hasattr(it, "reset") and getattr(it, "resetSupported", lambda: True)():
                it.reset()
            self._fire("onEpochStart")
            t0 = time.perf_counter()
            src = it
            depth = int(getattr(self, "asyncPrefetch", 2))
            if depth > 0 and getattr(it, "asyncSupported", lambda: False)() and not isinstance(it, AsyncDataSetIterator):
                src = AsyncDataSetIterator(it, depth, device=self.device)
            for ds in src:
                self._last_etl_ms = (time.perf_counter() - t0) * 1e3
                self._fit_batch(ds)
                t0 = time.perf_counter()
            if src is not it and hasattr(src, "shutdown"):
                src.shutdown()
            self._fire("onEpochEnd")
            self.incrementEpochCount()
        return self
