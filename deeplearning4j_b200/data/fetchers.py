"""Dataset iterators over the classic benchmark datasets (``deeplearning4j-datasets``: ``MnistDataSetIterator``,
``EmnistDataSetIterator``, ``Cifar10DataSetIterator``, ``IrisDataSetIterator``, ``TinyImageNetDataSetIterator``,
``SvhnDataSetIterator``, ``UciSequenceDataSetIterator``, ``LFWDataSetIterator``).

The reference downloads the archives on first use.  There is no network here, so every iterator reads the standard
files from a local directory (``DL4J_DATA_DIR`` or ``~/.deeplearning4j/data/<NAME>``) and raises ``FileNotFoundError``
naming the files it expects; ``synthetic=True`` instead generates a deterministic stand-in of the same shapes and label
space, which is what benchmarks and smoke tests use.  Iris ships inline (150 rows)."""
from __future__ import annotations

import gzip
import os
import pickle
import struct

import numpy as np
import torch

from .dataset import DataSet
from .iterators import DataSetIterator


def data_dir(name):
    root = os.environ.get("DL4J_DATA_DIR") or os.path.join(os.path.expanduser("~"), ".deeplearning4j", "data")
    return os.path.join(root, name)


class _ArrayIterator(DataSetIterator):
    def __init__(self, x, y, batch, num_classes=None, shuffle=False, seed=123, labels=None, one_hot=True):
        self.x, self.y, self.batchSize = x, y, int(batch)
        self.numClasses, self.shuffle, self.seed, self.labelNames = num_classes, shuffle, seed, labels
        self.one_hot = one_hot
        self.preProcessor = None
        self._epoch = 0
        self.reset()

    def reset(self):
        n = self.x.shape[0]
        if self.shuffle:
            g = torch.Generator().manual_seed(self.seed + self._epoch)
            self._order = torch.randperm(n, generator=g)
        else:
            self._order = torch.arange(n)
        self._epoch += 1
        self._pos = 0

    def hasNext(self): return self._pos < self.x.shape[0]
    def resetSupported(self): return True
    def asyncSupported(self): return True
    def batch(self): return self.batchSize
    def totalOutcomes(self): return self.numClasses
    def inputColumns(self): return int(np.prod(self.x.shape[1:]))
    def getLabels(self): return self.labelNames
    def setPreProcessor(self, p): self.preProcessor = p
    def getPreProcessor(self): return self.preProcessor
    def numExamples(self): return self.x.shape[0]
    totalExamples = numExamples

    def next(self, n=None):
        idx = self._order[self._pos:self._pos + (n or self.batchSize)]
        self._pos += idx.numel()
        x = self.x[idx].float()
        y = self.y[idx]
        if self.one_hot and self.numClasses and y.dim() == 1:
            y = torch.nn.functional.one_hot(y.long(), self.numClasses).float()
        ds = DataSet(x, y)
        if self.preProcessor is not None:
            self.preProcessor.preProcess(ds)
        return ds

    __next__ = next

    def __iter__(self):
        self.reset()
        while self.hasNext():
            yield self.next()


def _synthetic_images(n, shape, classes, seed):
    """Class-dependent blobs: learnable, deterministic, same dtype/range as the real pixels (0..255)."""
    g = torch.Generator().manual_seed(seed)
    y = torch.randint(0, classes, (n,), generator=g)
    protos = torch.rand(classes, *shape, generator=g)
    x = (0.6 * protos[y] + 0.4 * torch.rand(n, *shape, generator=g)) * 255.0
    return x.to(torch.uint8), y


def _read_idx(path):
    op = gzip.open if path.endswith(".gz") else open
    with op(path, "rb") as f:
        magic, = struct.unpack(">I", f.read(4))
        nd = magic & 0xFF
        dims = struct.unpack(">" + "I" * nd, f.read(4 * nd))
        return np.frombuffer(f.read(), dtype=np.uint8).reshape(dims)


def _find(directory, *cands):
    for c in cands:
        for ext in ("", ".gz"):
            p = os.path.join(directory, c + ext)
            if os.path.exists(p):
                return p
    raise FileNotFoundError(f"expected one of {list(cands)} (optionally .gz) under {directory}; datasets cannot be downloaded in this environment "
                            f"(pass synthetic=True for generated stand-in data)")


class MnistDataSetIterator(_ArrayIterator):
    """28x28 grey digits as flat [N, 784] rows scaled to 0..1 (``binarize`` thresholds at 0.5 like the reference)."""
    NAME, FILES = "MNIST", ("train-images-idx3-ubyte", "train-labels-idx1-ubyte", "t10k-images-idx3-ubyte", "t10k-labels-idx1-ubyte")

    def __init__(self, batch, train=True, seed=123, numExamples=None, binarize=False, shuffle=None, synthetic=False, path=None, classes=10):
        if synthetic:
            n = numExamples or (60000 if train else 10000)
            x, y = _synthetic_images(min(n, 8192), (28, 28), classes, seed + (0 if train else 1))
        else:
            d = path or data_dir(self.NAME)
            fi, fl = (self.FILES[0], self.FILES[1]) if train else (self.FILES[2], self.FILES[3])
            x = torch.from_numpy(_read_idx(_find(d, fi, fi.replace("-idx", ".idx"))).copy())
            y = torch.from_numpy(_read_idx(_find(d, fl, fl.replace("-idx", ".idx"))).copy()).long()
        if numExamples:
            x, y = x[:numExamples], y[:numExamples]
        x = x.reshape(x.shape[0], -1).float() / 255.0
        if binarize:
            x = (x > 0.5).float()
        super().__init__(x, y, batch, classes, train if shuffle is None else shuffle, seed, [str(i) for i in range(classes)])


class EmnistDataSetIterator(MnistDataSetIterator):
    class Set:
        COMPLETE, MERGE, BALANCED, LETTERS, DIGITS, MNIST = "byclass", "bymerge", "balanced", "letters", "digits", "mnist"
    NUM = {"byclass": 62, "bymerge": 47, "balanced": 47, "letters": 26, "digits": 10, "mnist": 10}

    def __init__(self, dataSet, batch, train=True, seed=123, synthetic=False, path=None, **kw):
        self.NAME = "EMNIST"
        t = "train" if train else "test"
        self.FILES = (f"emnist-{dataSet}-{t}-images-idx3-ubyte", f"emnist-{dataSet}-{t}-labels-idx1-ubyte") * 2
        super().__init__(batch, True, seed, synthetic=synthetic, path=path, classes=self.NUM[dataSet], shuffle=train, **kw)

    @staticmethod
    def numLabels(dataSet): return EmnistDataSetIterator.NUM[dataSet]


class Cifar10DataSetIterator(_ArrayIterator):
    """[N, 3, 32, 32] from the python-pickle batches (``cifar-10-batches-py``) or the binary ``data_batch_*.bin`` files."""
    LABELS = ["airplane", "automobile", "bird", "cat", "deer", "dog", "frog", "horse", "ship", "truck"]

    def __init__(self, batch, train=True, seed=123, numExamples=None, synthetic=False, path=None, shuffle=None):
        if synthetic:
            x, y = _synthetic_images(numExamples or 4096, (3, 32, 32), 10, seed + (0 if train else 1))
        else:
            d = path or data_dir("CIFAR10")
            names = [f"data_batch_{i}" for i in range(1, 6)] if train else ["test_batch"]
            xs, ys = [], []
            for nm in names:
                pb = os.path.join(d, nm + ".bin")
                pp = next((p for p in (os.path.join(d, nm), os.path.join(d, "cifar-10-batches-py", nm)) if os.path.exists(p)), None)
                if os.path.exists(pb):
                    raw = np.fromfile(pb, dtype=np.uint8).reshape(-1, 3073)
                    ys.append(raw[:, 0].astype(np.int64)); xs.append(raw[:, 1:].reshape(-1, 3, 32, 32))
                elif pp:
                    with open(pp, "rb") as f:
                        b = pickle.load(f, encoding="bytes")
                    xs.append(np.asarray(b[b"data"], dtype=np.uint8).reshape(-1, 3, 32, 32)); ys.append(np.asarray(b[b"labels"], dtype=np.int64))
                else:
                    raise FileNotFoundError(f"expected {nm}(.bin) under {d}; datasets cannot be downloaded in this environment (pass synthetic=True)")
            x, y = torch.from_numpy(np.concatenate(xs)), torch.from_numpy(np.concatenate(ys))
        if numExamples:
            x, y = x[:numExamples], y[:numExamples]
        super().__init__(x, y, batch, 10, train if shuffle is None else shuffle, seed, self.LABELS)


CifarDataSetIterator = Cifar10DataSetIterator


class _ImageFolderIterator(_ArrayIterator):
    """Datasets laid out as ``<root>/<split>/<label>/*.{ppm,pgm,npy,png,jpg}``."""

    def __init__(self, name, batch, shape, classes, train, seed, synthetic, path, numExamples=None):
        if synthetic:
            x, y = _synthetic_images(numExamples or 1024, shape, classes, seed + (0 if train else 1))
            labels = [str(i) for i in range(classes)]
        else:
            from ..datavec.records import FileSplit, ImageRecordReader, ParentPathLabelGenerator
            root = os.path.join(path or data_dir(name), "train" if train else "test")
            if not os.path.isdir(root):
                raise FileNotFoundError(f"expected an image folder tree at {root}; datasets cannot be downloaded in this environment (pass synthetic=True)")
            rr = ImageRecordReader(shape[1], shape[2], shape[0], ParentPathLabelGenerator()).initialize(FileSplit(root))
            xs, ys = zip(*[(r[0], r[1]) for r in rr])
            x, y, labels = torch.stack(xs), torch.tensor(ys), rr.getLabels()
        super().__init__(x, y, batch, classes, train, seed, labels)


class TinyImageNetDataSetIterator(_ImageFolderIterator):
    def __init__(self, batch, imgDim=(64, 64), train=True, seed=123, synthetic=False, path=None, numExamples=None):
        super().__init__("TINYIMAGENET", batch, (3, imgDim[0], imgDim[1]), 200, train, seed, synthetic, path, numExamples)


class SvhnDataSetIterator(_ImageFolderIterator):
    def __init__(self, batch, train=True, seed=123, synthetic=False, path=None, numExamples=None):
        super().__init__("SVHN", batch, (3, 32, 32), 10, train, seed, synthetic, path, numExamples)


class LFWDataSetIterator(_ImageFolderIterator):
    def __init__(self, batch, numExamples=None, imgDim=(3, 250, 250), numLabels=5749, train=True, seed=123, synthetic=False, path=None):
        super().__init__("LFW", batch, tuple(imgDim), numLabels, train, seed, synthetic, path, numExamples or 256)


class UciSequenceDataSetIterator(_ArrayIterator):
    """UCI synthetic-control time series: 600 sequences of length 60, 6 classes -> features [N, 1, 60], per-step labels."""

    def __init__(self, batch, train=True, seed=123, synthetic=False, path=None):
        if synthetic:
            g = torch.Generator().manual_seed(seed)
            y = torch.arange(600) // 100
            t = torch.arange(60.0)
            base = torch.stack([torch.zeros(60), 15 * torch.sin(2 * np.pi * t / 12), 0.4 * t, -0.4 * t, 10.0 * (t > 30), -10.0 * (t > 30)])
            x = 30 + base[y] + 2 * torch.randn(600, 60, generator=g)
        else:
            p = _find(path or data_dir("UCI"), "synthetic_control.data")
            x = torch.tensor(np.loadtxt(p), dtype=torch.float32)
            y = torch.arange(x.shape[0]) // 100
        g = torch.Generator().manual_seed(seed)
        perm = torch.randperm(x.shape[0], generator=g)
        cut = int(0.75 * x.shape[0])
        idx = perm[:cut] if train else perm[cut:]
        x, y = x[idx].unsqueeze(1), y[idx]
        yy = torch.nn.functional.one_hot(y, 6).float().unsqueeze(2).expand(-1, -1, 60).contiguous()
        super().__init__(x, yy, batch, 6, train, seed, ["normal", "cyclic", "increasing", "decreasing", "upward shift", "downward shift"], one_hot=False)


_IRIS = """5.1,3.5,1.4,0.2,0 4.9,3.0,1.4,0.2,0 4.7,3.2,1.3,0.2,0 4.6,3.1,1.5,0.2,0 5.0,3.6,1.4,0.2,0 5.4,3.9,1.7,0.4,0 4.6,3.4,1.4,0.3,0 5.0,3.4,1.5,0.2,0 4.4,2.9,1.4,0.2,0 4.9,3.1,1.5,0.1,0
5.4,3.7,1.5,0.2,0 4.8,3.4,1.6,0.2,0 4.8,3.0,1.4,0.1,0 4.3,3.0,1.1,0.1,0 5.8,4.0,1.2,0.2,0 5.7,4.4,1.5,0.4,0 5.4,3.9,1.3,0.4,0 5.1,3.5,1.4,0.3,0 5.7,3.8,1.7,0.3,0 5.1,3.8,1.5,0.3,0
5.4,3.4,1.7,0.2,0 5.1,3.7,1.5,0.4,0 4.6,3.6,1.0,0.2,0 5.1,3.3,1.7,0.5,0 4.8,3.4,1.9,0.2,0 5.0,3.0,1.6,0.2,0 5.0,3.4,1.6,0.4,0 5.2,3.5,1.5,0.2,0 5.2,3.4,1.4,0.2,0 4.7,3.2,1.6,0.2,0
4.8,3.1,1.6,0.2,0 5.4,3.4,1.5,0.4,0 5.2,4.1,1.5,0.1,0 5.5,4.2,1.4,0.2,0 4.9,3.1,1.5,0.1,0 5.0,3.2,1.2,0.2,0 5.5,3.5,1.3,0.2,0 4.9,3.1,1.5,0.1,0 4.4,3.0,1.3,0.2,0 5.1,3.4,1.5,0.2,0
5.0,3.5,1.3,0.3,0 4.5,2.3,1.3,0.3,0 4.4,3.2,1.3,0.2,0 5.0,3.5,1.6,0.6,0 5.1,3.8,1.9,0.4,0 4.8,3.0,1.4,0.3,0 5.1,3.8,1.6,0.2,0 4.6,3.2,1.4,0.2,0 5.3,3.7,1.5,0.2,0 5.0,3.3,1.4,0.2,0
7.0,3.2,4.7,1.4,1 6.4,3.2,4.5,1.5,1 6.9,3.1,4.9,1.5,1 5.5,2.3,4.0,1.3,1 6.5,2.8,4.6,1.5,1 5.7,2.8,4.5,1.3,1 6.3,3.3,4.7,1.6,1 4.9,2.4,3.3,1.0,1 6.6,2.9,4.6,1.3,1 5.2,2.7,3.9,1.4,1
5.0,2.0,3.5,1.0,1 5.9,3.0,4.2,1.5,1 6.0,2.2,4.0,1.0,1 6.1,2.9,4.7,1.4,1 5.6,2.9,3.6,1.3,1 6.7,3.1,4.4,1.4,1 5.6,3.0,4.5,1.5,1 5.8,2.7,4.1,1.0,1 6.2,2.2,4.5,1.5,1 5.6,2.5,3.9,1.1,1
5.9,3.2,4.8,1.8,1 6.1,2.8,4.0,1.3,1 6.3,2.5,4.9,1.5,1 6.1,2.8,4.7,1.2,1 6.4,2.9,4.3,1.3,1 6.6,3.0,4.4,1.4,1 6.8,2.8,4.8,1.4,1 6.7,3.0,5.0,1.7,1 6.0,2.9,4.5,1.5,1 5.7,2.6,3.5,1.0,1
5.5,2.4,3.8,1.1,1 5.5,2.4,3.7,1.0,1 5.8,2.7,3.9,1.2,1 6.0,2.7,5.1,1.6,1 5.4,3.0,4.5,1.5,1 6.0,3.4,4.5,1.6,1 6.7,3.1,4.7,1.5,1 6.3,2.3,4.4,1.3,1 5.6,3.0,4.1,1.3,1 5.5,2.5,4.0,1.3,1
5.5,2.6,4.4,1.2,1 6.1,3.0,4.6,1.4,1 5.8,2.6,4.0,1.2,1 5.0,2.3,3.3,1.0,1 5.6,2.7,4.2,1.3,1 5.7,3.0,4.2,1.2,1 5.7,2.9,4.2,1.3,1 6.2,2.9,4.3,1.3,1 5.1,2.5,3.0,1.1,1 5.7,2.8,4.1,1.3,1
6.3,3.3,6.0,2.5,2 5.8,2.7,5.1,1.9,2 7.1,3.0,5.9,2.1,2 6.3,2.9,5.6,1.8,2 6.5,3.0,5.8,2.2,2 7.6,3.0,6.6,2.1,2 4.9,2.5,4.5,1.7,2 7.3,2.9,6.3,1.8,2 6.7,2.5,5.8,1.8,2 7.2,3.6,6.1,2.5,2
6.5,3.2,5.1,2.0,2 6.4,2.7,5.3,1.9,2 6.8,3.0,5.5,2.1,2 5.7,2.5,5.0,2.0,2 5.8,2.8,5.1,2.4,2 6.4,3.2,5.3,2.3,2 6.5,3.0,5.5,1.8,2 7.7,3.8,6.7,2.2,2 7.7,2.6,6.9,2.3,2 6.0,2.2,5.0,1.5,2
6.9,3.2,5.7,2.3,2 5.6,2.8,4.9,2.0,2 7.7,2.8,6.7,2.0,2 6.3,2.7,4.9,1.8,2 6.7,3.3,5.7,2.1,2 7.2,3.2,6.0,1.8,2 6.2,2.8,4.8,1.8,2 6.1,3.0,4.9,1.8,2 6.4,2.8,5.6,2.1,2 7.2,3.0,5.8,1.6,2
7.4,2.8,6.1,1.9,2 7.9,3.8,6.4,2.0,2 6.4,2.8,5.6,2.2,2 6.3,2.8,5.1,1.5,2 6.1,2.6,5.6,1.4,2 7.7,3.0,6.1,2.3,2 6.3,3.4,5.6,2.4,2 6.4,3.1,5.5,1.8,2 6.0,3.0,4.8,1.8,2 6.9,3.1,5.4,2.1,2
6.7,3.1,5.6,2.4,2 6.9,3.1,5.1,2.3,2 5.8,2.7,5.1,1.9,2 6.8,3.2,5.9,2.3,2 6.7,3.3,5.7,2.5,2 6.7,3.0,5.2,2.3,2 6.3,2.5,5.0,1.9,2 6.5,3.0,5.2,2.0,2 6.2,3.4,5.4,2.3,2 5.9,3.0,5.1,1.8,2"""


class IrisDataSetIterator(_ArrayIterator):
    def __init__(self, batch=150, numExamples=150, shuffle=False, seed=123):
        rows = [[float(v) for v in tok.split(",")] for tok in _IRIS.split()]
        arr = torch.tensor(rows)[:numExamples]
        super().__init__(arr[:, :4], arr[:, 4].long(), batch, 3, shuffle, seed, ["Iris-setosa", "Iris-versicolor", "Iris-virginica"])
