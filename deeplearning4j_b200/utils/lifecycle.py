"""Allocation lifecycle tracking and leak reports.

Parity: libnd4j ``array/{NDArrayLifecycleTracker, DataBufferLifecycleTracker}``, ``helpers/{TADCacheLifecycleTracker,
ShapeCacheLifecycleTracker}`` and the Java ``DeallocatorService`` reports: every tracked object is recorded with its size,
kind and (optionally) the creating stack; live objects are found through weak references, so a report lists what is still
alive, grouped by allocation site, and a temporal report shows growth between two snapshots.
"""
from __future__ import annotations

import threading
import time
import traceback
import weakref
from collections import defaultdict


class LifecycleTracker:
    _instance = None

    def __init__(self, capture_stacks=False, stack_depth=8):
        self.capture_stacks, self.stack_depth = capture_stacks, stack_depth
        self._lock = threading.Lock()
        self._live = {}            # id -> (weakref, kind, bytes, site, time)
        self.total_allocations = 0
        self.total_bytes = 0
        self.enabled = False

    @classmethod
    def getInstance(cls):
        if cls._instance is None:
            cls._instance = LifecycleTracker()
        return cls._instance

    def enable(self, capture_stacks=False):
        self.enabled, self.capture_stacks = True, capture_stacks
        return self

    def disable(self):
        self.enabled = False

    def _site(self):
        if not self.capture_stacks:
            return "<stack capture off>"
        frames = traceback.extract_stack(limit=self.stack_depth + 3)[:-3]
        return " <- ".join(f"{f.filename.rsplit('/', 1)[-1]}:{f.lineno}" for f in reversed(frames[-self.stack_depth:]))

    def recordAllocation(self, obj, kind="NDArray", nbytes=None):
        if not self.enabled:
            return obj
        if nbytes is None:
            import torch
            t = obj if isinstance(obj, torch.Tensor) else getattr(obj, "t", None)
            nbytes = int(t.numel() * t.element_size()) if isinstance(t, torch.Tensor) else 0
        key = id(obj)
        site = self._site()

        def gone(_ref, key=key):
            with self._lock:
                self._live.pop(key, None)
        try:
            ref = weakref.ref(obj, gone)
        except TypeError:
            return obj
        with self._lock:
            self._live[key] = (ref, kind, nbytes, site, time.time())
            self.total_allocations += 1
            self.total_bytes += nbytes
        return obj

    def recordDeallocation(self, obj):
        with self._lock:
            self._live.pop(id(obj), None)

    def liveCount(self, kind=None):
        with self._lock:
            return sum(1 for _, k, *_ in self._live.values() if kind is None or k == kind)

    def liveBytes(self, kind=None):
        with self._lock:
            return sum(b for _, k, b, *_ in self._live.values() if kind is None or k == kind)

    def snapshot(self):
        with self._lock:
            by_site = defaultdict(lambda: [0, 0])
            for _, kind, nbytes, site, _t in self._live.values():
                e = by_site[(kind, site)]
                e[0] += 1
                e[1] += nbytes
            return {k: tuple(v) for k, v in by_site.items()}

    def generateLeakReport(self, top=20):
        snap = sorted(self.snapshot().items(), key=lambda kv: -kv[1][1])
        lines = [f"live objects: {self.liveCount()}  live bytes: {self.liveBytes()}  allocations seen: {self.total_allocations}"]
        for (kind, site), (n, b) in snap[:top]:
            lines.append(f"  {kind:12s} x{n:<6d} {b:>14d} B  {site}")
        return "\n".join(lines)

    @staticmethod
    def temporalReport(before, after, top=20):
        """Growth between two ``snapshot()`` results (allocation sites whose live bytes increased)."""
        grow = []
        for k, (n, b) in after.items():
            n0, b0 = before.get(k, (0, 0))
            if b > b0:
                grow.append((b - b0, n - n0, k))
        grow.sort(reverse=True)
        return [f"+{db} B (+{dn} objects) {kind} {site}" for db, dn, (kind, site) in grow[:top]]

    def reset(self):
        with self._lock:
            self._live.clear()
            self.total_allocations = self.total_bytes = 0
