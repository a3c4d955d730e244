"""``ParallelInference`` (``deeplearning4j-parallelwrapper/.../parallelism/ParallelInference.java:54-690``)
and ``InplaceParallelInference``.

One worker thread per replica; each worker owns a model replica on its device and a CUDA stream, so
requests on different replicas overlap.  ``InferenceMode.BATCHED`` coalesces queued requests (up to
``batchLimit`` examples) into one forward pass and scatters the rows back to the callers' futures —
the micro-batching the reference does with ``ObservablesProvider`` (``:644-690``).  ``SEQUENTIAL`` runs
one request per forward pass; ``INPLACE`` runs the forward pass on the calling thread against a replica
chosen by the load balancer (no queue hop).
"""
from __future__ import annotations

import itertools
import queue
import threading
from concurrent.futures import Future

import torch

from ..nd.ndarray import INDArray


class InferenceMode:
    SEQUENTIAL = "SEQUENTIAL"
    BATCHED = "BATCHED"
    INPLACE = "INPLACE"


class LoadBalanceMode:
    ROUND_ROBIN = "ROUND_ROBIN"
    FIFO = "FIFO"


def _t(x):
    return x.t if isinstance(x, INDArray) else (x if isinstance(x, torch.Tensor) else torch.as_tensor(x))


class _Request:
    __slots__ = ("x", "mask", "future", "n")

    def __init__(self, x, mask):
        self.x, self.mask, self.future, self.n = x, mask, Future(), x.shape[0]


class _Worker(threading.Thread):
    def __init__(self, pi, idx, model, device, q):
        super().__init__(daemon=True, name=f"InferenceWorker-{idx}")
        self.pi, self.idx, self.model, self.device, self.q = pi, idx, model, device, q
        self.stream = torch.cuda.Stream(device) if device.type == "cuda" else None
        self.processed = 0
        self.batches = 0
        self._halt = threading.Event()

    def _forward(self, x, mask):
        with torch.no_grad():
            if self.stream is not None:
                with torch.cuda.stream(self.stream):
                    out = self.model.output(x.to(self.device, non_blocking=True), False, None if mask is None else mask.to(self.device))
                    out = _t(out[0] if isinstance(out, (list, tuple)) else out)
                self.stream.synchronize()
                return out
            out = self.model.output(x, False, mask)
            return _t(out[0] if isinstance(out, (list, tuple)) else out)

    def run(self):
        pi = self.pi
        while not self._halt.is_set():
            try:
                first = self.q.get(timeout=0.05)
            except queue.Empty:
                continue
            if first is None:
                break
            batch = [first]
            if pi.inferenceMode == InferenceMode.BATCHED:
                total = first.n
                while total < pi.batchLimit:
                    try:
                        nxt = self.q.get_nowait()
                    except queue.Empty:
                        break
                    if nxt is None:
                        self._halt.set()
                        break
                    # only requests of the same trailing shape (and mask presence) can share a forward pass
                    if nxt.x.shape[1:] != first.x.shape[1:] or (nxt.mask is None) != (first.mask is None):
                        self.q.put(nxt)
                        break
                    batch.append(nxt)
                    total += nxt.n
            try:
                if len(batch) == 1:
                    outs = [self._forward(first.x, first.mask)]
                else:
                    x = torch.cat([r.x for r in batch], 0)
                    m = None if first.mask is None else torch.cat([r.mask for r in batch], 0)
                    out = self._forward(x, m)
                    outs, o = [], 0
                    for r in batch:
                        outs.append(out[o:o + r.n])
                        o += r.n
                for r, o in zip(batch, outs):
                    r.future.set_result(INDArray(o))
                self.processed += sum(r.n for r in batch)
                self.batches += 1
            except Exception as e:                                  # noqa: BLE001 - delivered to the callers
                for r in batch:
                    if not r.future.done():
                        r.future.set_exception(e)

    def shutdown(self):
        self._halt.set()


class ParallelInference:
    def __init__(self, model, workers=None, inferenceMode=InferenceMode.BATCHED, batchLimit=32, queueLimit=64,
                 loadBalanceMode=LoadBalanceMode.FIFO, devices=None):
        self.inferenceMode, self.batchLimit, self.queueLimit, self.loadBalanceMode = inferenceMode, int(batchLimit), int(queueLimit), loadBalanceMode
        if devices is None:
            n_gpu = torch.cuda.device_count() if torch.cuda.is_available() and model.device.type == "cuda" else 0
            devices = [torch.device("cuda", i) for i in range(n_gpu)] or [model.device]
        workers = workers or len(devices)
        self.devices = [torch.device(devices[i % len(devices)]) for i in range(workers)]
        self.model = model
        self.replicas = []
        for d in self.devices:
            self.replicas.append(model if d == model.device and not self.replicas else self._replicate(model, d))
        shared = queue.Queue(self.queueLimit) if loadBalanceMode == LoadBalanceMode.FIFO else None
        self.queues = [shared or queue.Queue(self.queueLimit) for _ in self.devices]
        self._rr = itertools.count()
        self.workers = []
        if inferenceMode != InferenceMode.INPLACE:
            for i, (m, d, q) in enumerate(zip(self.replicas, self.devices, self.queues)):
                w = _Worker(self, i, m, d, q)
                w.start()
                self.workers.append(w)
        self._locks = [threading.Lock() for _ in self.devices]

    @staticmethod
    def _replicate(model, device):
        r = model.clone() if device == model.device else None
        if r is None:
            r = type(model)(model.conf.clone())
            r.device = device
            r.init(model.params().t.to(device) if hasattr(model.params(), "t") else model.params().to(device), False)
        return r

    class Builder:
        def __init__(self, model): self.model, self.kw = model, {}
        def workers(self, n): self.kw["workers"] = n; return self
        def inferenceMode(self, m): self.kw["inferenceMode"] = m; return self
        def batchLimit(self, n): self.kw["batchLimit"] = n; return self
        def queueLimit(self, n): self.kw["queueLimit"] = n; return self
        def loadBalanceMode(self, m): self.kw["loadBalanceMode"] = m; return self
        def devices(self, d): self.kw["devices"] = d; return self
        def build(self): return ParallelInference(self.model, **self.kw)

    def updateModel(self, model):
        """Swap in new parameters on every replica (``ParallelInference.updateModel``)."""
        p = model.params()
        p = p.t if hasattr(p, "t") and not isinstance(p, torch.Tensor) else p
        for r, lock in zip(self.replicas, self._locks):
            with lock:
                r.setParams(p.to(r.device))
        self.model = model

    def getCurrentModelsFromWorkers(self): return list(self.replicas)

    def outputAsync(self, x, mask=None):
        x = _t(x)
        req = _Request(x, None if mask is None else _t(mask))
        i = next(self._rr) % len(self.queues)
        self.queues[i].put(req)
        return req.future

    def output(self, x, mask=None):
        if self.inferenceMode == InferenceMode.INPLACE:
            i = next(self._rr) % len(self.replicas)
            with self._locks[i], torch.no_grad():
                r = self.replicas[i]
                out = r.output(_t(x).to(r.device), False, None if mask is None else _t(mask).to(r.device))
                return out[0] if isinstance(out, (list, tuple)) else out
        return self.outputAsync(x, mask).result()

    def outputBatches(self, xs):
        futs = [self.outputAsync(x) for x in xs]
        return [f.result() for f in futs]

    def stats(self):
        return [{"worker": w.idx, "device": str(w.device), "examples": w.processed, "batches": w.batches} for w in self.workers]

    def shutdown(self):
        for w in self.workers:
            w.shutdown()
        for q in set(self.queues):
            for _ in self.workers:
                try:
                    q.put_nowait(None)
                except queue.Full:
                    pass
        for w in self.workers:
            w.join(timeout=2.0)


class InplaceParallelInference(ParallelInference):
    def __init__(self, model, **kw):
        kw["inferenceMode"] = InferenceMode.INPLACE
        super().__init__(model, **kw)
