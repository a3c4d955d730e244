"""DataSet iterators (``nd4j-api/.../linalg/dataset/api/iterator`` and
``deeplearning4j-data/deeplearning4j-utility-iterators``).

``AsyncDataSetIterator`` is the B200 version of the reference's prefetch thread
(``AsyncDataSetIterator.java:366-460``): a background thread pulls batches, pins them in host
memory and issues the host->device copy on a dedicated CUDA stream, so the training stream only
waits on an event.
"""
from __future__ import annotations

import queue
import threading
from typing import Callable, Iterable

import torch

from .dataset import DataSet, MultiDataSet


class DataSetIterator:
    """Base class: Python iteration protocol plus the DL4J ``hasNext/next/reset`` surface."""
    preProcessor = None

    def hasNext(self) -> bool: raise NotImplementedError
    def next(self, num=None): raise NotImplementedError
    def reset(self): pass
    def resetSupported(self): return True
    def asyncSupported(self): return True
    def batch(self): return -1
    def inputColumns(self): return -1
    def totalOutcomes(self): return -1
    def getLabels(self): return None
    def setPreProcessor(self, p): self.preProcessor = p
    def getPreProcessor(self): return self.preProcessor

    def _pp(self, ds):
        if self.preProcessor is not None and ds is not None:
            self.preProcessor.preProcess(ds)
        return ds

    def __iter__(self):
        return self

    def __next__(self):
        if not self.hasNext():
            raise StopIteration
        return self.next()


MultiDataSetIterator = DataSetIterator


class ListDataSetIterator(DataSetIterator):
    def __init__(self, data, batch=None):
        if isinstance(data, DataSet):
            data = data.asList() if batch else [data]
        self.data = list(data)
        self._batch = batch or 1 if batch else None
        self.pos = 0

    def hasNext(self): return self.pos < len(self.data)

    def next(self, num=None):
        if self._batch:
            chunk = self.data[self.pos:self.pos + self._batch]
            self.pos += len(chunk)
            return self._pp(DataSet.merge(chunk))
        d = self.data[self.pos]
        self.pos += 1
        return self._pp(d)

    def reset(self): self.pos = 0
    def batch(self): return self._batch or -1
    def inputColumns(self): return self.data[0].numInputs()
    def totalOutcomes(self): return self.data[0].numOutcomes()


class INDArrayDataSetIterator(DataSetIterator):
    """Batches over in-memory feature/label arrays."""
    def __init__(self, features, labels, batch, featuresMask=None, labelsMask=None):
        self.ds = DataSet(features, labels, featuresMask, labelsMask)
        self._batch, self.pos = int(batch), 0

    def hasNext(self): return self.pos < self.ds.numExamples()

    def next(self, num=None):
        n = num or self._batch
        d = self.ds.getRange(self.pos, min(self.pos + n, self.ds.numExamples()))
        self.pos += d.numExamples()
        return self._pp(d)

    def reset(self): self.pos = 0
    def batch(self): return self._batch
    def inputColumns(self): return self.ds.numInputs()
    def totalOutcomes(self): return self.ds.numOutcomes()


ViewIterator = INDArrayDataSetIterator
DoublesDataSetIterator = FloatsDataSetIterator = INDArrayDataSetIterator


class ExistingDataSetIterator(DataSetIterator):
    def __init__(self, iterable: Iterable):
        self.src, self.it, self._peek = iterable, None, None
        self.reset()

    def reset(self):
        self.it = iter(self.src)
        self._peek = None

    def hasNext(self):
        if self._peek is None:
            try:
                self._peek = next(self.it)
            except StopIteration:
                return False
        return True

    def next(self, num=None):
        if not self.hasNext():
            raise StopIteration
        d, self._peek = self._peek, None
        return self._pp(d)

    def resetSupported(self):
        return not hasattr(self.src, "__next__")


IteratorDataSetIterator = ExistingDataSetIterator


class _Wrapping(DataSetIterator):
    def __init__(self, base):
        self.base = base
    def hasNext(self): return self.base.hasNext()
    def next(self, num=None): return self._pp(self.base.next())
    def reset(self): self.base.reset()
    def resetSupported(self): return self.base.resetSupported()
    def asyncSupported(self): return self.base.asyncSupported()
    def batch(self): return self.base.batch()
    def inputColumns(self): return self.base.inputColumns()
    def totalOutcomes(self): return self.base.totalOutcomes()
    def getLabels(self): return self.base.getLabels()


class EarlyTerminationDataSetIterator(_Wrapping):
    def __init__(self, base, terminationPoint):
        super().__init__(base)
        self.limit, self.count = int(terminationPoint), 0
    def hasNext(self): return self.count < self.limit and self.base.hasNext()
    def next(self, num=None):
        self.count += 1
        return super().next()
    def reset(self):
        self.count = 0
        self.base.reset()


EarlyTerminationMultiDataSetIterator = EarlyTerminationDataSetIterator


class MultipleEpochsIterator(_Wrapping):
    def __init__(self, numEpochs, base):
        super().__init__(base)
        self.numEpochs, self.epoch = int(numEpochs), 0
    def hasNext(self):
        if self.base.hasNext():
            return True
        if self.epoch + 1 < self.numEpochs:
            self.epoch += 1
            self.base.reset()
            return self.base.hasNext()
        return False
    def reset(self):
        self.epoch = 0
        self.base.reset()


class SamplingDataSetIterator(DataSetIterator):
    def __init__(self, sampleFrom: DataSet, batchSize, totalNumberSamples, seed=None):
        self.ds, self.bs, self.total, self.done, self.seed = sampleFrom, batchSize, totalNumberSamples, 0, seed
    def hasNext(self): return self.done < self.total
    def next(self, num=None):
        self.done += self.bs
        return self._pp(self.ds.sample(self.bs, withReplacement=True))
    def reset(self): self.done = 0


class BenchmarkDataSetIterator(DataSetIterator):
    """Synthetic fixed-shape batches, generated once and re-served (``BenchmarkDataSetIterator.java``)."""
    def __init__(self, featuresShape, numLabels, totalIterations, labelsShape=None, seed=12345, device="cpu", dtype=torch.float32):
        g = torch.Generator().manual_seed(seed)
        f = torch.rand(tuple(featuresShape), generator=g).to(dtype)
        if labelsShape is not None:
            l = torch.rand(tuple(labelsShape), generator=g).to(dtype)
        else:
            idx = torch.randint(0, numLabels, (featuresShape[0],), generator=g)
            l = torch.nn.functional.one_hot(idx, numLabels).to(dtype)
        self.ds = DataSet(f.to(device), l.to(device))
        self.limit, self.count = int(totalIterations), 0
    def hasNext(self): return self.count < self.limit
    def next(self, num=None):
        self.count += 1
        return self.ds
    def reset(self): self.count = 0
    def asyncSupported(self): return False


class RandomDataSetIterator(DataSetIterator):
    class Values:
        RANDOM_UNIFORM = "RANDOM_UNIFORM"; RANDOM_NORMAL = "RANDOM_NORMAL"; ONE_HOT = "ONE_HOT"
        ZEROS = "ZEROS"; ONES = "ONES"; BINARY = "BINARY"; INTEGER_0_10 = "INTEGER_0_10"
        INTEGER_0_100 = "INTEGER_0_100"; INTEGER_0_1000 = "INTEGER_0_1000"

    def __init__(self, numMiniBatches, featuresShape, labelsShape, featureValues="RANDOM_UNIFORM", labelValues="ONE_HOT", seed=0):
        self.n, self.fs, self.ls, self.fv, self.lv = numMiniBatches, tuple(featuresShape), tuple(labelsShape), featureValues, labelValues
        self.g = torch.Generator().manual_seed(seed)
        self.count = 0

    def _gen(self, shape, kind):
        if kind == "RANDOM_UNIFORM": return torch.rand(shape, generator=self.g)
        if kind == "RANDOM_NORMAL": return torch.randn(shape, generator=self.g)
        if kind == "ZEROS": return torch.zeros(shape)
        if kind == "ONES": return torch.ones(shape)
        if kind == "BINARY": return (torch.rand(shape, generator=self.g) < 0.5).float()
        if kind.startswith("INTEGER_0_"): return torch.randint(0, int(kind.rsplit("_", 1)[1]), shape, generator=self.g).float()
        if kind == "ONE_HOT":
            idx = torch.randint(0, shape[1], (shape[0],) + tuple(shape[2:]), generator=self.g)
            oh = torch.nn.functional.one_hot(idx, shape[1]).float()
            return oh.movedim(-1, 1) if len(shape) > 2 else oh
        raise ValueError(kind)

    def hasNext(self): return self.count < self.n
    def next(self, num=None):
        self.count += 1
        return self._pp(DataSet(self._gen(self.fs, self.fv), self._gen(self.ls, self.lv)))
    def reset(self): self.count = 0


class MultiDataSetIteratorAdapter(_Wrapping):
    """DataSetIterator -> MultiDataSet stream."""
    def next(self, num=None):
        d = self.base.next()
        return MultiDataSet([d.features], [d.labels],
                            None if d.featuresMask is None else [d.featuresMask],
                            None if d.labelsMask is None else [d.labelsMask])


class MultiDataSetWrapperIterator(_Wrapping):
    """MultiDataSetIterator with one input/output -> DataSet stream."""
    def next(self, num=None):
        m = self.base.next()
        return self._pp(DataSet(m.features[0], m.labels[0], m.getFeaturesMaskArray(0) if m.featuresMasks else None,
                                m.getLabelsMaskArray(0) if m.labelsMasks else None))


class JointParallelDataSetIterator(DataSetIterator):
    """Round-robins over several iterators (``JointParallelDataSetIterator.java``)."""
    def __init__(self, *its, stop_on_first=True):
        self.its, self.i, self.stop_on_first = list(its), 0, stop_on_first
    def hasNext(self):
        if self.stop_on_first:
            return all(it.hasNext() for it in self.its)
        return any(it.hasNext() for it in self.its)
    def next(self, num=None):
        for _ in range(len(self.its)):
            it = self.its[self.i % len(self.its)]
            self.i += 1
            if it.hasNext():
                return self._pp(it.next())
        raise StopIteration
    def reset(self):
        self.i = 0
        for it in self.its:
            it.reset()


class DataSetIteratorSplitter:
    """Splits one iterator into train/test views by batch count (``DataSetIteratorSplitter.java``)."""
    def __init__(self, base, totalBatches, ratio):
        self.base, self.total, self.nTrain = base, int(totalBatches), int(totalBatches * ratio)
    def getTrainIterator(self):
        return _RangeIter(self.base, 0, self.nTrain)
    def getTestIterator(self):
        return _RangeIter(self.base, self.nTrain, self.total)


class _RangeIter(DataSetIterator):
    def __init__(self, base, a, b):
        self.base, self.a, self.b, self.pos = base, a, b, None
    def reset(self):
        self.base.reset()
        self.pos = 0
        while self.pos < self.a and self.base.hasNext():
            self.base.next()
            self.pos += 1
    def hasNext(self):
        if self.pos is None:
            self.reset()
        return self.pos < self.b and self.base.hasNext()
    def next(self, num=None):
        self.pos += 1
        return self._pp(self.base.next())


class AsyncShieldDataSetIterator(_Wrapping):
    """Marks the wrapped iterator as not to be wrapped in an async prefetcher."""
    def asyncSupported(self): return False


AsyncShieldMultiDataSetIterator = AsyncShieldDataSetIterator


class AsyncDataSetIterator(DataSetIterator):
    _END = object()

    def __init__(self, base, queueSize=2, device=None, pin=True):
        self.base, self.qsize = base, max(int(queueSize), 1)
        self.device = torch.device(device) if device is not None else None
        self.pin = pin and torch.cuda.is_available()
        self._q: queue.Queue | None = None
        self._thread = None
        self._peek = None
        self._err = None
        self._stop = threading.Event()
        self._stream = None
        self._start()

    def _start(self):
        self._stop.clear()
        self._q = queue.Queue(self.qsize)
        self._peek, self._err = None, None
        cuda = self.device is not None and self.device.type == "cuda"
        if cuda and self._stream is None:
            self._stream = torch.cuda.Stream(self.device)
        q, stop = self._q, self._stop

        def run():
            try:
                if cuda:
                    torch.cuda.set_device(self.device)
                while not stop.is_set() and self.base.hasNext():
                    d = self.base.next()
                    ev = None
                    if cuda:
                        d = d.pin() if self.pin else d
                        with torch.cuda.stream(self._stream):
                            d = d.to(self.device, non_blocking=True)
                            ev = torch.cuda.Event()
                            ev.record(self._stream)
                    while not stop.is_set():
                        try:
                            q.put((d, ev), timeout=0.1)
                            break
                        except queue.Full:
                            continue
            except BaseException as e:   # surfaced on the consumer side
                self._err = e
            finally:
                while True:
                    try:
                        q.put((AsyncDataSetIterator._END, None), timeout=0.1)
                        break
                    except queue.Full:
                        if stop.is_set():
                            break
        self._thread = threading.Thread(target=run, daemon=True, name="dl4j-async-prefetch")
        self._thread.start()

    def hasNext(self):
        if self._peek is None:
            self._peek = self._q.get()
        if self._peek[0] is AsyncDataSetIterator._END:
            if self._err is not None:
                e, self._err = self._err, None
                raise e
            return False
        return True

    def next(self, num=None):
        if not self.hasNext():
            raise StopIteration
        (d, ev), self._peek = self._peek, None
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)
        return self._pp(d)

    def shutdown(self):
        self._stop.set()
        if self._thread is not None:
            while self._thread.is_alive():
                try:
                    self._q.get_nowait()
                except queue.Empty:
                    pass
                self._thread.join(timeout=0.05)
            self._thread = None

    def reset(self):
        self.shutdown()
        self.base.reset()
        self._start()

    def resetSupported(self): return self.base.resetSupported()
    def asyncSupported(self): return False
    def batch(self): return self.base.batch()


AsyncMultiDataSetIterator = AsyncDataSetIterator
