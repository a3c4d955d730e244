"""``DataSet`` / ``MultiDataSet`` containers (``nd4j-api/.../linalg/dataset/DataSet.java``,
``MultiDataSet.java``): features, labels and optional mask arrays, with the reference's
utility surface (split, shuffle, batchBy, merge, save/load, normalisation helpers)."""
from __future__ import annotations

import io
import struct

import numpy as np
import torch

from ..nd.ndarray import INDArray, _unwrap, wrap


def _t(x):
    if x is None:
        return None
    x = _unwrap(x)
    return x if isinstance(x, torch.Tensor) else torch.as_tensor(np.asarray(x))


class DataSet:
    def __init__(self, features=None, labels=None, featuresMask=None, labelsMask=None):
        self.features, self.labels = _t(features), _t(labels)
        self.featuresMask, self.labelsMask = _t(featuresMask), _t(labelsMask)
        self.exampleMetaData = None
        self.labelNames = None

    # accessors (tensors are returned raw: layers consume torch tensors directly)
    def getFeatures(self): return self.features
    def getLabels(self): return self.labels
    def getFeaturesMaskArray(self): return self.featuresMask
    def getLabelsMaskArray(self): return self.labelsMask
    def setFeatures(self, f): self.features = _t(f)
    def setLabels(self, l): self.labels = _t(l)
    def setFeaturesMaskArray(self, m): self.featuresMask = _t(m)
    def setLabelsMaskArray(self, m): self.labelsMask = _t(m)
    def hasMaskArrays(self): return self.featuresMask is not None or self.labelsMask is not None
    def numExamples(self): return 0 if self.features is None else int(self.features.shape[0])
    def numInputs(self): return int(self.features.shape[1])
    def numOutcomes(self): return int(self.labels.shape[1])
    def isEmpty(self): return self.features is None
    def getExampleMetaData(self): return self.exampleMetaData
    def setExampleMetaData(self, m): self.exampleMetaData = m
    def getLabelNamesList(self): return self.labelNames
    def setLabelNames(self, n): self.labelNames = list(n)
    def __len__(self): return self.numExamples()

    def to(self, device, non_blocking=True):
        mv = lambda t: None if t is None else t.to(device, non_blocking=non_blocking)
        return DataSet(mv(self.features), mv(self.labels), mv(self.featuresMask), mv(self.labelsMask))

    def pin(self):
        pn = lambda t: None if t is None else (t if t.is_cuda or t.is_pinned() or not torch.cuda.is_available() else t.pin_memory())
        return DataSet(pn(self.features), pn(self.labels), pn(self.featuresMask), pn(self.labelsMask))

    def copy(self):
        c = lambda t: None if t is None else t.clone()
        return DataSet(c(self.features), c(self.labels), c(self.featuresMask), c(self.labelsMask))

    def get(self, i):
        idx = [i] if isinstance(i, int) else list(i)
        g = lambda t: None if t is None else t[idx]
        return DataSet(g(self.features), g(self.labels), g(self.featuresMask), g(self.labelsMask))

    def getRange(self, a, b):
        g = lambda t: None if t is None else t[a:b]
        return DataSet(g(self.features), g(self.labels), g(self.featuresMask), g(self.labelsMask))

    def asList(self):
        return [self.get(i) for i in range(self.numExamples())]

    def batchBy(self, n):
        return [self.getRange(i, min(i + n, self.numExamples())) for i in range(0, self.numExamples(), n)]

    def shuffle(self, seed=None):
        g = torch.Generator().manual_seed(seed) if seed is not None else None
        perm = torch.randperm(self.numExamples(), generator=g)
        for a in ("features", "labels", "featuresMask", "labelsMask"):
            t = getattr(self, a)
            if t is not None:
                setattr(self, a, t[perm.to(t.device)])

    def splitTestAndTrain(self, n_or_frac, seed=None):
        n = int(n_or_frac * self.numExamples()) if isinstance(n_or_frac, float) and n_or_frac < 1 else int(n_or_frac)
        return SplitTestAndTrain(self.getRange(0, n), self.getRange(n, self.numExamples()))

    def sample(self, n, seed=None, withReplacement=False):
        g = torch.Generator().manual_seed(seed) if seed is not None else None
        idx = (torch.randint(0, self.numExamples(), (n,), generator=g) if withReplacement
               else torch.randperm(self.numExamples(), generator=g)[:n])
        return self.get(idx.tolist())

    def filterBy(self, labels):
        keep = [i for i in range(self.numExamples()) if int(self.labels[i].argmax()) in labels]
        return self.get(keep)

    def scale(self):
        mx = self.features.abs().max()
        self.features = self.features / mx

    def scaleMinAndMax(self, lo, hi):
        mn, mx = self.features.amin(0, keepdim=True), self.features.amax(0, keepdim=True)
        self.features = (self.features - mn) / (mx - mn).clamp_min(1e-12) * (hi - lo) + lo

    def normalizeZeroMeanZeroUnitVariance(self):
        self.features = (self.features - self.features.mean(0, keepdim=True)) / self.features.std(0, keepdim=True).clamp_min(1e-12)

    def binarize(self, cutoff=0.0):
        self.features = (self.features > cutoff).to(self.features.dtype)

    def addFeatureVector(self, v):
        self.features = torch.cat([self.features, _t(v).reshape(1, -1)], 0)

    def outcome(self):
        return int(self.labels.reshape(-1).argmax())

    @staticmethod
    def merge(datasets):
        datasets = list(datasets)
        if not datasets:
            return DataSet()
        f0 = datasets[0].features
        if f0.dim() == 3 and len({d.features.shape[2] for d in datasets}) > 1:
            return _merge_time_series(datasets)
        cat = lambda xs: None if xs[0] is None else torch.cat(xs, 0)
        return DataSet(cat([d.features for d in datasets]), cat([d.labels for d in datasets]),
                       cat([d.featuresMask for d in datasets]), cat([d.labelsMask for d in datasets]))

    # binary save/load: ND4J array streams back to back, preceded by a presence bitmask
    def save(self, path_or_stream):
        from ..serde.binary import write_array
        own = isinstance(path_or_stream, str)
        f = open(path_or_stream, "wb") if own else path_or_stream
        arrs = [self.features, self.labels, self.featuresMask, self.labelsMask]
        f.write(struct.pack(">B", sum((1 << i) for i, a in enumerate(arrs) if a is not None)))
        for a in arrs:
            if a is not None:
                write_array(INDArray(a), f)
        if own:
            f.close()

    @staticmethod
    def load(path_or_stream):
        from ..serde.binary import read_array
        own = isinstance(path_or_stream, str)
        f = open(path_or_stream, "rb") if own else path_or_stream
        (bits,) = struct.unpack(">B", f.read(1))
        arrs = [read_array(f).t if bits & (1 << i) else None for i in range(4)]
        if own:
            f.close()
        return DataSet(*arrs)

    def __repr__(self):
        sh = lambda t: None if t is None else list(t.shape)
        return f"DataSet(features={sh(self.features)}, labels={sh(self.labels)}, fmask={sh(self.featuresMask)}, lmask={sh(self.labelsMask)})"


def _merge_time_series(datasets):
    T = max(d.features.shape[2] for d in datasets)
    fs, ls, fm, lm = [], [], [], []
    for d in datasets:
        t = d.features.shape[2]
        pad = T - t
        fs.append(torch.nn.functional.pad(d.features, [0, pad]))
        ls.append(torch.nn.functional.pad(d.labels, [0, pad]) if d.labels.dim() == 3 else d.labels)
        m = d.featuresMask if d.featuresMask is not None else torch.ones(d.features.shape[0], t)
        fm.append(torch.nn.functional.pad(m, [0, pad]))
        m2 = d.labelsMask if d.labelsMask is not None else torch.ones(d.features.shape[0], t)
        lm.append(torch.nn.functional.pad(m2, [0, pad]))
    return DataSet(torch.cat(fs), torch.cat(ls), torch.cat(fm), torch.cat(lm))


class SplitTestAndTrain:
    def __init__(self, train, test):
        self.train, self.test = train, test
    def getTrain(self): return self.train
    def getTest(self): return self.test


class MultiDataSet:
    def __init__(self, features=None, labels=None, featuresMasks=None, labelsMasks=None):
        lst = lambda v: None if v is None else ([_t(e) for e in v] if isinstance(v, (list, tuple)) else [_t(v)])
        self.features, self.labels = lst(features) or [], lst(labels) or []
        self.featuresMasks, self.labelsMasks = lst(featuresMasks), lst(labelsMasks)

    def getFeatures(self, i=None): return self.features if i is None else self.features[i]
    def getLabels(self, i=None): return self.labels if i is None else self.labels[i]
    def getFeaturesMaskArrays(self): return self.featuresMasks
    def getLabelsMaskArrays(self): return self.labelsMasks
    def getFeaturesMaskArray(self, i): return None if self.featuresMasks is None else self.featuresMasks[i]
    def getLabelsMaskArray(self, i): return None if self.labelsMasks is None else self.labelsMasks[i]
    def numFeatureArrays(self): return len(self.features)
    def numLabelsArrays(self): return len(self.labels)
    def setFeatures(self, *a):
        if len(a) == 2: self.features[a[0]] = _t(a[1])
        else: self.features = [_t(e) for e in a[0]]
    def setLabels(self, *a):
        if len(a) == 2: self.labels[a[0]] = _t(a[1])
        else: self.labels = [_t(e) for e in a[0]]
    def setFeaturesMaskArrays(self, m): self.featuresMasks = None if m is None else [_t(e) for e in m]
    def setLabelsMaskArrays(self, m): self.labelsMasks = None if m is None else [_t(e) for e in m]
    def hasMaskArrays(self): return self.featuresMasks is not None or self.labelsMasks is not None
    def numExamples(self): return int(self.features[0].shape[0]) if self.features else 0

    def to(self, device, non_blocking=True):
        mv = lambda v: None if v is None else [None if t is None else t.to(device, non_blocking=non_blocking) for t in v]
        return MultiDataSet(mv(self.features), mv(self.labels), mv(self.featuresMasks), mv(self.labelsMasks))

    def pin(self):
        ok = torch.cuda.is_available()
        pn = lambda v: None if v is None else [None if t is None else (t.pin_memory() if ok and not t.is_cuda and not t.is_pinned() else t) for t in v]
        return MultiDataSet(pn(self.features), pn(self.labels), pn(self.featuresMasks), pn(self.labelsMasks))

    @staticmethod
    def merge(mds):
        mds = list(mds)
        cat = lambda i, attr: torch.cat([getattr(m, attr)[i] for m in mds], 0)
        f = [cat(i, "features") for i in range(len(mds[0].features))]
        l = [cat(i, "labels") for i in range(len(mds[0].labels))]
        fm = None if mds[0].featuresMasks is None else [cat(i, "featuresMasks") for i in range(len(mds[0].featuresMasks))]
        lm = None if mds[0].labelsMasks is None else [cat(i, "labelsMasks") for i in range(len(mds[0].labelsMasks))]
        return MultiDataSet(f, l, fm, lm)

    def asList(self):
        n = self.numExamples()
        g = lambda v, i: None if v is None else [None if t is None else t[i:i + 1] for t in v]
        return [MultiDataSet(g(self.features, i), g(self.labels, i), g(self.featuresMasks, i), g(self.labelsMasks, i)) for i in range(n)]

    def save(self, path):
        from ..serde.binary import write_array
        with open(path, "wb") as f:
            groups = [self.features, self.labels, self.featuresMasks or [], self.labelsMasks or []]
            f.write(struct.pack(">4i", *[len(g) for g in groups]))
            for g in groups:
                for a in g:
                    f.write(struct.pack(">B", 0 if a is None else 1))
                    if a is not None:
                        write_array(INDArray(a), f)

    @staticmethod
    def load(path):
        from ..serde.binary import read_array
        with open(path, "rb") as f:
            counts = struct.unpack(">4i", f.read(16))
            groups = []
            for c in counts:
                g = []
                for _ in range(c):
                    (has,) = struct.unpack(">B", f.read(1))
                    g.append(read_array(f).t if has else None)
                groups.append(g)
        return MultiDataSet(groups[0], groups[1], groups[2] or None, groups[3] or None)
