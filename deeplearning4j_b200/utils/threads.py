"""Host-side parallel loops (libnd4j ``execution/Threads.h``: ``parallel_for``, ``parallel_tad``, ``parallel_do``,
``parallel_long`` / ``parallel_double`` reductions over a pooled set of workers).  Used by the CPU data path (record
readers, image decoding, host-side codecs); tensor math itself runs on torch's own intra-op pool."""
from __future__ import annotations

import os
from concurrent.futures import ThreadPoolExecutor

_POOL = None


def max_threads():
    from .environment import Environment
    n = Environment.getInstance().maxThreads() if hasattr(Environment.getInstance(), "maxThreads") else 0
    return int(n) if n else (os.cpu_count() or 1)


def _pool():
    global _POOL
    if _POOL is None:
        _POOL = ThreadPoolExecutor(max_workers=max_threads(), thread_name_prefix="dl4j-worker")
    return _POOL


def _spans(start, stop, step, n_threads):
    total = max(0, (stop - start + step - 1) // step)
    n = max(1, min(n_threads, total))
    per = (total + n - 1) // n
    out = []
    for t in range(n):
        a = start + t * per * step
        b = min(stop, a + per * step)
        if a < b:
            out.append((a, b))
    return out


def parallel_for(fn, start, stop, step=1, numThreads=None):
    """``fn(thread_id, start, stop, step)`` over disjoint spans; returns the number of spans used."""
    spans = _spans(start, stop, step, numThreads or max_threads())
    if len(spans) <= 1:
        for i, (a, b) in enumerate(spans):
            fn(i, a, b, step)
        return len(spans)
    list(_pool().map(lambda iab: fn(iab[0], iab[1][0], iab[1][1], step), enumerate(spans)))
    return len(spans)


parallel_tad = parallel_for


def parallel_do(fn, numThreads=None):
    """``fn(thread_id, num_threads)`` once per worker."""
    n = numThreads or max_threads()
    list(_pool().map(lambda i: fn(i, n), range(n)))
    return n


def _reduce(fn, combine, start, stop, step, numThreads):
    spans = _spans(start, stop, step, numThreads or max_threads())
    parts = list(_pool().map(lambda iab: fn(iab[0], iab[1][0], iab[1][1], step), enumerate(spans))) if len(spans) > 1 \
        else [fn(i, a, b, step) for i, (a, b) in enumerate(spans)]
    acc = None
    for p in parts:
        acc = p if acc is None else combine(acc, p)
    return acc


def parallel_long(fn, combine, start, stop, step=1, numThreads=None):
    r = _reduce(fn, combine, start, stop, step, numThreads)
    return int(r) if r is not None else 0


def parallel_double(fn, combine, start, stop, step=1, numThreads=None):
    r = _reduce(fn, combine, start, stop, step, numThreads)
    return float(r) if r is not None else 0.0
