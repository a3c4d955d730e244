"""The remaining utility iterators of ``deeplearning4j-utility-iterators`` (``org.deeplearning4j.datasets.iterator.**``): adapters over
plain Python iterators and number pairs, file-backed iterators, singleton / dummy-block / reconstruction / scrollable / joint
iterators, multi-dataset forms of the wrapping iterators, and the callbacks of the parallel iterators."""
from __future__ import annotations

import os
import threading
from queue import Queue

import torch

from .dataset import DataSet, MultiDataSet
from .iterators import DataSetIterator, _Wrapping


class AbstractDataSetIterator(DataSetIterator):
    """Batches an iterable of (features, labels) pairs (``AbstractDataSetIterator.java``); ``FloatsDataSetIterator`` /
    ``DoublesDataSetIterator`` / ``INDArrayDataSetIterator`` are this class with a fixed element type."""

    dtype = None

    def __init__(self, iterable, batchSize):
        self.iterable, self.batchSize = iterable, int(batchSize)
        self._it = None

    def reset(self): self._it = iter(self.iterable)
    def batch(self): return self.batchSize

    def _fill(self):
        if self._it is None:
            self.reset()
        if getattr(self, "_peek", None) is None:
            self._peek = next(self._it, None)

    def hasNext(self):
        self._fill()
        return self._peek is not None

    def next(self, num=None):
        self._fill()
        fs, ls = [], []
        while self._peek is not None and len(fs) < (num or self.batchSize):
            f, l = self._peek
            fs.append(torch.as_tensor(f, dtype=self.dtype).reshape(-1) if self.dtype is not None else torch.as_tensor(f))
            ls.append(torch.as_tensor(l, dtype=self.dtype).reshape(-1) if self.dtype is not None else torch.as_tensor(l))
            self._peek = next(self._it, None)
        return self._pp(DataSet(torch.stack(fs), torch.stack(ls)))


class FloatsDataSetIterator(AbstractDataSetIterator):
    dtype = torch.float32


class DoublesDataSetIterator(AbstractDataSetIterator):
    dtype = torch.float64


class IteratorDataSetIterator(DataSetIterator):
    """Re-batches an iterator of DataSets of any size into batches of ``batchSize`` examples (``IteratorDataSetIterator.java``)."""

    def __init__(self, iterator, batchSize):
        self.src, self.batchSize = iterator, int(batchSize)
        self._it, self._rest = None, None

    def reset(self):
        if hasattr(self.src, "reset"):
            self.src.reset()
        self._it, self._rest = iter(self.src), None

    def resetSupported(self): return hasattr(self.src, "reset") or not hasattr(self.src, "__next__")

    def _more(self):
        if self._it is None:
            self._it = iter(self.src)
        return next(self._it, None)

    def hasNext(self):
        if self._rest is not None and self._rest.numExamples() > 0:
            return True
        self._rest = self._more()
        return self._rest is not None

    def next(self, num=None):
        n = num or self.batchSize
        parts, have = [], 0
        while have < n and self.hasNext():
            d, self._rest = self._rest, None
            take = min(n - have, d.numExamples())
            if take < d.numExamples():
                self._rest = DataSet(d.features[take:], d.labels[take:])
                d = DataSet(d.features[:take], d.labels[:take])
            parts.append(d)
            have += take
        return self._pp(DataSet.merge(parts) if len(parts) > 1 else parts[0])

    def batch(self): return self.batchSize


class IteratorMultiDataSetIterator(IteratorDataSetIterator):
    def next(self, num=None):
        n = num or self.batchSize
        parts, have = [], 0
        while have < n and self.hasNext():
            d, self._rest = self._rest, None
            parts.append(d)
            have += d.features[0].shape[0]
        if len(parts) == 1:
            return parts[0]
        cat = lambda k: [torch.cat([getattr(p, k)[i] for p in parts]) for i in range(len(getattr(parts[0], k)))]
        return MultiDataSet(cat("features"), cat("labels"))

    def hasNext(self):
        if self._rest is not None:
            return True
        self._rest = self._more()
        return self._rest is not None


class SingletonDataSetIterator(DataSetIterator):
    def __init__(self, ds): self.ds, self._done = ds, False
    def reset(self): self._done = False
    def hasNext(self): return not self._done
    def next(self, num=None):
        self._done = True
        return self._pp(self.ds)


SingletonMultiDataSetIterator = SingletonDataSetIterator


class DummyBlockDataSetIterator(_Wrapping):
    """``next(n)`` returns up to n DataSets at once (``BlockDataSetIterator``)."""
    def hasAnything(self): return self.base.hasNext()
    def next(self, num=None):
        if num is None:
            return self._pp(self.base.next())
        out = []
        while len(out) < num and self.base.hasNext():
            out.append(self._pp(self.base.next()))
        return out


DummyBlockMultiDataSetIterator = DummyBlockDataSetIterator


class DummyPreProcessor:
    def preProcess(self, ds): return None


class CombinedPreProcessor:
    """Applies several pre-processors in order (``CombinedPreProcessor.Builder``)."""
    def __init__(self, *pps): self.pps = list(pps)

    class Builder:
        def __init__(self): self.items = {}
        def addPreProcessor(self, *a):
            (idx, pp) = a if len(a) == 2 else (len(self.items), a[0])
            self.items[int(idx)] = pp
            return self
        def build(self): return CombinedPreProcessor(*[self.items[k] for k in sorted(self.items)])

    def preProcess(self, ds):
        for p in self.pps:
            p.preProcess(ds)


CombinedMultiDataSetPreProcessor = CombinedPreProcessor


class ReconstructionDataSetIterator(_Wrapping):
    """Labels := features (auto-encoder training)."""
    def next(self, num=None):
        d = self.base.next()
        return self._pp(DataSet(d.features, d.features.clone()))


class ScrollableDataSetIterator(DataSetIterator):
    """A window [start, start + count) of batches over a backing iterator, used by ``DataSetIteratorSplitter``-style partitions."""
    def __init__(self, num, backing, counter=None, resetPending=None, firstTrain=None, ratio=None, totalBatches=None):
        self.backing = backing
        total = int(totalBatches) if totalBatches is not None else None
        if ratio is not None and total is not None:
            n_train = int(total * ratio)
            self.start, self.count = (0, n_train) if num == 0 else (n_train, total - n_train)
        else:
            self.start, self.count = 0, total
        self._pos = None

    def reset(self):
        self.backing.reset()
        for _ in range(self.start):
            if self.backing.hasNext():
                self.backing.next()
        self._pos = 0

    def hasNext(self):
        if self._pos is None:
            self.reset()
        return (self.count is None or self._pos < self.count) and self.backing.hasNext()

    def next(self, num=None):
        if self._pos is None:
            self.reset()
        self._pos += 1
        return self._pp(self.backing.next())


ScrollableMultiDataSetIterator = ScrollableDataSetIterator


class MultiDataSetIteratorSplitter:
    def __init__(self, base, totalBatches, ratio): self.base, self.total, self.ratio = base, int(totalBatches), float(ratio)
    def getTrainIterator(self): return ScrollableDataSetIterator(0, self.base, ratio=self.ratio, totalBatches=self.total)
    def getTestIterator(self): return ScrollableDataSetIterator(1, self.base, ratio=self.ratio, totalBatches=self.total)


class EarlyTerminationMultiDataSetIterator(_Wrapping):
    def __init__(self, it, terminationPoint):
        super().__init__(it)
        if terminationPoint <= 0:
            raise ValueError("Termination point (the number of calls to .next() or .next(num)) has to be > 0")
        self.limit, self.n = int(terminationPoint), 0
    def reset(self): self.base.reset(); self.n = 0
    def hasNext(self): return self.n < self.limit and self.base.hasNext()
    def next(self, num=None):
        self.n += 1
        return self._pp(self.base.next())


class JointMultiDataSetIterator(DataSetIterator):
    """Several DataSetIterators stepped together; their features (and the labels of ``outcome`` or of all) form one MultiDataSet."""
    def __init__(self, *iterators, outcome=-1):
        self.its, self.outcome = list(iterators), int(outcome)
    def reset(self): [i.reset() for i in self.its]
    def hasNext(self): return all(i.hasNext() for i in self.its)
    def next(self, num=None):
        ds = [i.next() for i in self.its]
        feats = [d.features for d in ds]
        labels = [d.labels for d in ds] if self.outcome < 0 else [ds[self.outcome].labels]
        return self._pp(MultiDataSet(feats, labels))


class RandomMultiDataSetIterator(DataSetIterator):
    """``numMiniBatches`` MultiDataSets of random arrays; per array a shape and a value kind (``RandomMultiDataSetIterator.Values``)."""
    ZEROS, ONES, RANDOM_UNIFORM, RANDOM_NORMAL, ONE_HOT, INTEGER_0_10, INTEGER_0_100 = range(7)

    class Builder:
        def __init__(self, numMiniBatches): self.n, self.f, self.l, self.seed = int(numMiniBatches), [], [], 0
        def addFeatures(self, shape, values=2): self.f.append((tuple(shape), values)); return self
        def addLabels(self, shape, values=4): self.l.append((tuple(shape), values)); return self
        def setSeed(self, s): self.seed = int(s); return self
        def build(self): return RandomMultiDataSetIterator(self.n, self.f, self.l, self.seed)

    def __init__(self, numMiniBatches, features, labels, seed=0):
        self.n, self.f, self.l, self.seed = int(numMiniBatches), list(features), list(labels), int(seed)
        self.reset()

    def reset(self): self.i, self.g = 0, torch.Generator().manual_seed(self.seed)
    def hasNext(self): return self.i < self.n

    def _make(self, shape, kind):
        if kind == self.ZEROS: return torch.zeros(shape)
        if kind == self.ONES: return torch.ones(shape)
        if kind == self.RANDOM_UNIFORM: return torch.rand(shape, generator=self.g)
        if kind == self.RANDOM_NORMAL: return torch.randn(shape, generator=self.g)
        if kind == self.ONE_HOT:
            idx = torch.randint(0, shape[-1], shape[:-1], generator=self.g)
            return torch.nn.functional.one_hot(idx, shape[-1]).float()
        hi = 10 if kind == self.INTEGER_0_10 else 100
        return torch.randint(0, hi, shape, generator=self.g).float()

    def next(self, num=None):
        self.i += 1
        return self._pp(MultiDataSet([self._make(*s) for s in self.f], [self._make(*s) for s in self.l]))


class BenchmarkMultiDataSetIterator(DataSetIterator):
    """The same MultiDataSet ``limit`` times (no allocation per step)."""
    def __init__(self, featureShapes, numLabels, totalIterations):
        g = torch.Generator().manual_seed(0)
        feats = [torch.rand(tuple(s), generator=g) for s in featureShapes]
        labs = [torch.nn.functional.one_hot(torch.randint(0, n, (feats[0].shape[0],), generator=g), n).float() for n in numLabels]
        self.mds, self.limit, self.i = MultiDataSet(feats, labs), int(totalIterations), 0
    def reset(self): self.i = 0
    def hasNext(self): return self.i < self.limit
    def next(self, num=None):
        self.i += 1
        return self.mds


class AsyncMultiDataSetIterator(DataSetIterator):
    """Prefetches from the wrapped iterator on a background thread (queue of ``queueSize``)."""
    _END = object()

    def __init__(self, it, queueSize=2):
        self.it, self.size = it, max(int(queueSize), 1)
        self._start()

    def _start(self):
        self.q = Queue(self.size)
        self._peek = None

        def run():
            try:
                while self.it.hasNext():
                    self.q.put(self.it.next())
            finally:
                self.q.put(self._END)
        self.t = threading.Thread(target=run, daemon=True)
        self.t.start()

    def reset(self):
        self.shutdown()
        self.it.reset()
        self._start()

    def shutdown(self):
        while self.t.is_alive():
            try:
                self.q.get(timeout=0.05)
            except Exception:       # noqa: BLE001
                pass

    def hasNext(self):
        if self._peek is None:
            self._peek = self.q.get()
        return self._peek is not self._END

    def next(self, num=None):
        if not self.hasNext():
            raise StopIteration
        v, self._peek = self._peek, None
        return self._pp(v)


class AsyncShieldMultiDataSetIterator(_Wrapping):
    def asyncSupported(self): return False
    def next(self, num=None): return self._pp(self.base.next())


class WorkspacesShieldDataSetIterator(_Wrapping):
    """Detaches every DataSet from the workspace it was created in (tensors here are never workspace-bound: a pass-through that
    clones, so that the consumer owns its arrays)."""
    def next(self, num=None):
        d = self.base.next()
        return self._pp(DataSet(d.features.clone(), None if d.labels is None else d.labels.clone()))


# --------------------------------------------------------------------------------------------------------- file-backed iterators
class BaseFileIterator(DataSetIterator):
    """Iterates over saved DataSet / MultiDataSet files under one or more directories (``file/BaseFileIterator.java``): optional
    extension filter, shuffling by seed, and re-batching to ``batchSize`` examples."""

    def __init__(self, roots, recursive=True, randomSeed=None, batchSize=-1, validExtensions=None):
        roots = [roots] if isinstance(roots, (str, os.PathLike)) else list(roots)
        files = []
        for r in roots:
            if os.path.isfile(r):
                files.append(os.fspath(r))
                continue
            for base, _, names in os.walk(r):
                files += [os.path.join(base, n) for n in sorted(names)]
                if not recursive:
                    break
        if validExtensions:
            files = [f for f in files if f.rsplit(".", 1)[-1] in set(validExtensions)]
        self.files, self.seed, self.batchSize = sorted(files), randomSeed, int(batchSize)
        self.reset()

    def _load(self, path): raise NotImplementedError
    def _merge(self, parts): raise NotImplementedError
    def _size(self, d): raise NotImplementedError
    def _split(self, d, n): raise NotImplementedError

    def reset(self):
        order = list(range(len(self.files)))
        if self.seed is not None:
            g = torch.Generator().manual_seed(int(self.seed))
            order = torch.randperm(len(order), generator=g).tolist()
        self._order, self._pos, self._rest = order, 0, None

    def hasNext(self): return self._rest is not None or self._pos < len(self._order)

    def _next_file(self):
        d = self._load(self.files[self._order[self._pos]])
        self._pos += 1
        return d

    def next(self, num=None):
        if self.batchSize <= 0:
            return self._pp(self._next_file())
        parts, have = [], 0
        while have < self.batchSize and self.hasNext():
            d, self._rest = (self._rest, None) if self._rest is not None else (self._next_file(), None)
            take = min(self.batchSize - have, self._size(d))
            if take < self._size(d):
                d, self._rest = self._split(d, take)
            parts.append(d)
            have += take
        return self._pp(self._merge(parts) if len(parts) > 1 else parts[0])


class FileDataSetIterator(BaseFileIterator):
    def _load(self, path): return DataSet.load(path)
    def _merge(self, parts): return DataSet.merge(parts)
    def _size(self, d): return d.numExamples()
    def _split(self, d, n): return DataSet(d.features[:n], d.labels[:n]), DataSet(d.features[n:], d.labels[n:])


class FileMultiDataSetIterator(BaseFileIterator):
    def _load(self, path): return MultiDataSet.load(path)
    def _size(self, d): return d.features[0].shape[0]
    def _merge(self, parts):
        cat = lambda k: [torch.cat([getattr(p, k)[i] for p in parts]) for i in range(len(getattr(parts[0], k)))]
        return MultiDataSet(cat("features"), cat("labels"))
    def _split(self, d, n):
        return (MultiDataSet([f[:n] for f in d.features], [l[:n] for l in d.labels]),
                MultiDataSet([f[n:] for f in d.features], [l[n:] for l in d.labels]))


class FileSplitDataSetIterator(DataSetIterator):
    """One DataSet per file, produced by a callback (``FileSplitDataSetIterator`` + ``callbacks/FileCallback``)."""
    def __init__(self, files, callback):
        self.files, self.cb, self.i = list(files), callback, 0
    def reset(self): self.i = 0
    def hasNext(self): return self.i < len(self.files)
    def next(self, num=None):
        f = self.files[self.i]
        self.i += 1
        return self._pp(self.cb(f) if callable(self.cb) else self.cb.call(f))


class DataSetLoaderIterator(DataSetIterator):
    """Sources (paths, keys, ...) turned into DataSets by a loader function (``loader/DataSetLoaderIterator.java``)."""
    def __init__(self, sources, loader, shuffleSeed=None):
        self.src, self.loader, self.seed = list(sources), loader, shuffleSeed
        self.reset()
    def reset(self):
        self.order = list(range(len(self.src)))
        if self.seed is not None:
            self.order = torch.randperm(len(self.src), generator=torch.Generator().manual_seed(int(self.seed))).tolist()
        self.i = 0
    def hasNext(self): return self.i < len(self.order)
    def next(self, num=None):
        s = self.src[self.order[self.i]]
        self.i += 1
        return self._pp(self.loader(s) if callable(self.loader) else self.loader.load(s))


MultiDataSetLoaderIterator = DataSetLoaderIterator


# --------------------------------------------------------------------------------------------------------- callbacks
class DataSetCallback:
    def call(self, ds): return None
    def reset(self): return None


class DefaultCallback(DataSetCallback):
    """Makes sure the arrays of a prefetched DataSet live on the consumer's device before it is handed over."""
    def __init__(self, device=None): self.device = device
    def call(self, ds):
        if self.device is not None:
            ds.features = ds.features.to(self.device, non_blocking=True)
            if ds.labels is not None:
                ds.labels = ds.labels.to(self.device, non_blocking=True)


class InterleavedDataSetCallback(DataSetCallback):
    """Round-robin placement of consecutive DataSets on the devices (``InterleavedDataSetCallback``): DataSet k goes to device k mod n."""
    def __init__(self, devices=None):
        self.devices = list(devices) if devices is not None else [torch.device("cuda", i) for i in range(torch.cuda.device_count())] or [torch.device("cpu")]
        self.k = 0
    def call(self, ds):
        DefaultCallback(self.devices[self.k % len(self.devices)]).call(ds)
        self.k += 1
    def reset(self): self.k = 0


class FileCallback:
    def call(self, file): raise NotImplementedError


class DataSetDeserializer(FileCallback):
    def call(self, file): return DataSet.load(os.fspath(file))


class MultiBoolean:
    """A fixed-size set of flags with all-true / all-false queries (``parallel/MultiBoolean.java``)."""
    def __init__(self, numEntries, initialValue=False, oneTime=False):
        if numEntries > 32:
            raise ValueError("Too many entries: MultiBoolean holds at most 32")
        self.n, self.oneTime = int(numEntries), bool(oneTime)
        self.bits = (1 << self.n) - 1 if initialValue else 0
        self.touched = 0
    def set(self, value, entry):
        if entry < 0 or entry >= self.n:
            raise IndexError(f"entry {entry} out of {self.n}")
        if self.oneTime and (self.touched >> entry) & 1:
            return
        self.touched |= 1 << entry
        self.bits = self.bits | (1 << entry) if value else self.bits & ~(1 << entry)
    def allTrue(self): return self.bits == (1 << self.n) - 1
    def allFalse(self): return self.bits == 0


class FileSplitParallelDataSetIterator(DataSetIterator):
    """Files matching a pattern under a root, split between ``numThreads`` producers whose DataSets are interleaved in order."""
    def __init__(self, rootFolder, pattern, callback, numThreads=2, bufferPerThread=2):
        import fnmatch
        files = sorted(os.path.join(b, n) for b, _, ns in os.walk(rootFolder) for n in ns if fnmatch.fnmatch(n, pattern))
        if not files:
            raise ValueError(f"No files matching {pattern!r} under {rootFolder}")
        self.parts = [files[i::int(numThreads)] for i in range(int(numThreads))]
        self.cb, self.buf = callback, int(bufferPerThread)
        self.reset()
    def reset(self):
        self.its = [AsyncMultiDataSetIterator(FileSplitDataSetIterator(p, self.cb), self.buf) for p in self.parts if p]
        self.k = 0
    def hasNext(self): return any(i.hasNext() for i in self.its)
    def next(self, num=None):
        for _ in range(len(self.its)):
            it = self.its[self.k % len(self.its)]
            self.k += 1
            if it.hasNext():
                return self._pp(it.next())
        raise StopIteration
