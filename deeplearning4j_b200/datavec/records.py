"""DataVec records: writables, input splits, record readers and the bridge to DataSets
(``datavec-api/.../api/{writable,split,records/reader/impl}``, ``deeplearning4j-datavec-iterators``:
``RecordReaderDataSetIterator``, ``SequenceRecordReaderDataSetIterator``).

Writables are plain Python values (int / float / str / tensor); the typed ``*Writable`` classes exist for API
parity and carry their value in ``.value``.  Batches are assembled on the host into pinned memory when CUDA is
present, so the training loop's asynchronous prefetcher can copy them without a staging copy.
"""
from __future__ import annotations

import csv
import glob as _glob
import io
import json
import os
import random
import re

import numpy as np
import torch

from ..data.dataset import DataSet


# ----------------------------------------------------------------------------- writables
class Writable:
    def __init__(self, value): self.value = value
    def get(self): return self.value
    def toDouble(self): return float(self.value)
    def toFloat(self): return float(self.value)
    def toInt(self): return int(float(self.value))
    def toLong(self): return int(float(self.value))
    def toString(self): return str(self.value)
    __str__ = toString
    def __repr__(self): return f"{type(self).__name__}({self.value!r})"
    def __eq__(self, o): return (o.value if isinstance(o, Writable) else o) == self.value
    def __hash__(self): return hash(self.value)


class IntWritable(Writable): pass
class LongWritable(Writable): pass
class FloatWritable(Writable): pass
class DoubleWritable(Writable): pass
class BooleanWritable(Writable): pass
class Text(Writable): pass
class NullWritable(Writable):
    def __init__(self): super().__init__(None)
class NDArrayWritable(Writable):
    def toDouble(self): return float(self.value.reshape(-1)[0])
class BytesWritable(Writable): pass


def unwrap(v):
    return v.value if isinstance(v, Writable) else v


def _parse(tok):
    try:
        return int(tok)
    except ValueError:
        try:
            return float(tok)
        except ValueError:
            return tok


# ----------------------------------------------------------------------------- input splits
class InputSplit:
    def locations(self): raise NotImplementedError
    def length(self): return len(self.locations())


class FileSplit(InputSplit):
    def __init__(self, root, allowFormats=None, recursive=True, rng=None):
        self.root, self.allow, self.recursive, self.rng = str(root), allowFormats, recursive, rng
    def locations(self):
        if os.path.isfile(self.root):
            return [self.root]
        out = []
        for r, _, fs in os.walk(self.root):
            for f in sorted(fs):
                if self.allow is None or f.rsplit(".", 1)[-1].lower() in {a.lower().lstrip(".") for a in self.allow}:
                    out.append(os.path.join(r, f))
            if not self.recursive:
                break
        out.sort()
        if self.rng is not None:
            self.rng.shuffle(out)
        return out


class CollectionInputSplit(InputSplit):
    def __init__(self, uris): self.uris = [str(u) for u in uris]
    def locations(self): return list(self.uris)


class NumberedFileInputSplit(InputSplit):
    def __init__(self, baseString, minIdx, maxIdx): self.base, self.lo, self.hi = baseString, minIdx, maxIdx
    def locations(self): return [self.base % i for i in range(self.lo, self.hi + 1)]


class StringSplit(InputSplit):
    def __init__(self, data): self.data = data
    def locations(self): return [self.data]


class ListStringSplit(InputSplit):
    def __init__(self, data): self.data = list(data)
    def locations(self): return self.data


# ----------------------------------------------------------------------------- label generators
class ParentPathLabelGenerator:
    def getLabelForPath(self, path): return os.path.basename(os.path.dirname(str(path)))


class PatternPathLabelGenerator:
    def __init__(self, pattern, patternPosition=0): self.pattern, self.pos = pattern, patternPosition
    def getLabelForPath(self, path): return re.split(self.pattern, os.path.basename(str(path)))[self.pos]


# ----------------------------------------------------------------------------- record readers
class RecordReader:
    def initialize(self, split, conf=None):
        self.split = split
        self.reset()
        return self
    def hasNext(self): raise NotImplementedError
    def next(self): raise NotImplementedError
    def reset(self): raise NotImplementedError
    def getLabels(self): return None
    def resetSupported(self): return True
    def close(self): pass
    def __iter__(self):
        self.reset()
        while self.hasNext():
            yield self.next()
    def nextBatch(self, n):
        out = []
        while self.hasNext() and len(out) < n:
            out.append(self.next())
        return out


class _LineSource(RecordReader):
    def _lines(self):
        sp = self.split
        if isinstance(sp, StringSplit):
            yield from sp.data.splitlines()
        elif isinstance(sp, ListStringSplit):
            for item in sp.data:
                yield item
        else:
            for p in sp.locations():
                with open(p, encoding="utf-8", errors="replace", newline="") as f:
                    for line in f:
                        yield line.rstrip("\r\n")
    def reset(self):
        self._it = self._lines()
        self._skip()
        self._peek = next(self._it, None)
    def _skip(self): pass
    def hasNext(self): return self._peek is not None
    def _advance(self):
        v = self._peek
        self._peek = next(self._it, None)
        return v


class LineRecordReader(_LineSource):
    def next(self): return [self._advance()]


class CSVRecordReader(_LineSource):
    def __init__(self, skipNumLines=0, delimiter=",", quote='"'):
        self.skip, self.delim, self.quote = skipNumLines, delimiter, quote
    def _skip(self):
        for _ in range(self.skip):
            next(self._it, None)
    def _split(self, line):
        if isinstance(line, (list, tuple)):
            return [_parse(str(t)) for t in line]
        if self.quote and self.quote in line:
            return [_parse(t) for t in next(csv.reader([line], delimiter=self.delim, quotechar=self.quote))]
        return [_parse(t) for t in line.split(self.delim)]
    def next(self):
        line = self._advance()
        while line is not None and isinstance(line, str) and line.strip() == "" and self._peek is not None:
            line = self._advance()
        return self._split(line)


class CSVSequenceRecordReader(RecordReader):
    """One file = one sequence; every line one time step."""
    def __init__(self, skipNumLines=0, delimiter=","): self.skip, self.delim = skipNumLines, delimiter
    def reset(self):
        self._files = self.split.locations()
        self._i = 0
    def hasNext(self): return self._i < len(self._files)
    def sequenceRecord(self):
        p = self._files[self._i]
        self._i += 1
        with open(p) as f:
            lines = [l.rstrip("\r\n") for l in f][self.skip:]
        return [[_parse(t) for t in l.split(self.delim)] for l in lines if l != ""]
    next = sequenceRecord


class CSVRegexRecordReader(CSVRecordReader):
    def __init__(self, skipNumLines=0, delimiter=",", regexs=None):
        super().__init__(skipNumLines, delimiter)
        self.regexs = regexs or []
    def next(self):
        vals = super().next()
        out = []
        for v, rx in zip(vals, self.regexs + [None] * len(vals)):
            if rx is None:
                out.append(v)
            else:
                m = re.match(rx, str(v))
                out.extend(_parse(g) for g in m.groups()) if m else out.append(v)
        return out


class RegexLineRecordReader(_LineSource):
    def __init__(self, regex, skipNumLines=0): self.rx, self.skip = re.compile(regex), skipNumLines
    def _skip(self):
        for _ in range(self.skip):
            next(self._it, None)
    def next(self):
        line = self._advance()
        m = self.rx.match(line)
        if not m:
            raise ValueError(f"Invalid line: line does not match regex: {line!r}")
        return [_parse(g) for g in m.groups()]


class CollectionRecordReader(RecordReader):
    def __init__(self, records): self.records = [list(r) for r in records]
    def initialize(self, split=None, conf=None):
        self.reset()
        return self
    def reset(self): self._i = 0
    def hasNext(self): return self._i < len(self.records)
    def next(self):
        r = self.records[self._i]
        self._i += 1
        return [unwrap(v) for v in r]

InMemoryRecordReader = CollectionRecordReader


class CollectionSequenceRecordReader(CollectionRecordReader):
    def next(self):
        r = self.records[self._i]
        self._i += 1
        return [[unwrap(v) for v in step] for step in r]
    sequenceRecord = next


class JacksonLineRecordReader(_LineSource):
    """One JSON object per line; ``fields`` lists the (possibly nested, ``a/b``) keys to extract."""
    def __init__(self, fields, default=None): self.fields, self.default = list(fields), default
    def next(self):
        obj = json.loads(self._advance())
        out = []
        for fpath in self.fields:
            cur = obj
            for k in fpath.split("/"):
                cur = cur.get(k, self.default) if isinstance(cur, dict) else self.default
            out.append(cur)
        return out


class FileRecordReader(RecordReader):
    """Each file's whole content is one record (``[content]``, plus the parent-directory label index when labels exist)."""
    def __init__(self, appendLabel=False): self.appendLabel = appendLabel
    def reset(self):
        self._files = self.split.locations()
        self.labels = sorted({os.path.basename(os.path.dirname(p)) for p in self._files})
        self._i = 0
    def getLabels(self): return self.labels
    def hasNext(self): return self._i < len(self._files)
    def next(self):
        p = self._files[self._i]
        self._i += 1
        rec = [open(p, encoding="utf-8", errors="replace").read()]
        if self.appendLabel:
            rec.append(self.labels.index(os.path.basename(os.path.dirname(p))))
        return rec


class SVMLightRecordReader(_LineSource):
    """``label idx:value idx:value ...`` lines -> dense feature vector + label (``misc/SVMLightRecordReader.java``)."""
    def __init__(self, numFeatures, zeroBasedIndexing=False): self.n, self.zero = numFeatures, zeroBasedIndexing
    def next(self):
        parts = self._advance().split("#")[0].split()
        vec = [0.0] * self.n
        for kv in parts[1:]:
            k, v = kv.split(":")
            vec[int(k) - (0 if self.zero else 1)] = float(v)
        return vec + [_parse(parts[0])]


class ImageRecordReader(RecordReader):
    """Image files -> [C,H,W] float tensors (+ label index from the path).  Decodes PPM/PGM and ``.npy`` natively and
    other formats through PIL when it is installed (``datavec-data-image``: ``ImageRecordReader`` / ``NativeImageLoader``)."""

    def __init__(self, height, width, channels=3, labelGenerator=None):
        self.h, self.w, self.c, self.labelGen = height, width, channels, labelGenerator
        self.labels = []

    def reset(self):
        self._files = self.split.locations()
        if self.labelGen is not None:
            self.labels = sorted({self.labelGen.getLabelForPath(p) for p in self._files})
        self._i = 0

    def getLabels(self): return self.labels
    def hasNext(self): return self._i < len(self._files)

    @staticmethod
    def _read_pnm(raw):
        toks, pos = [], 0
        while len(toks) < 4:
            m = re.compile(rb"\s*(#[^\n]*\n\s*)*(\S+)").match(raw, pos)
            toks.append(m.group(2))
            pos = m.end()
            if toks[0] in (b"P4",) and len(toks) == 3:
                break
        magic, w, h = toks[0], int(toks[1]), int(toks[2])
        maxv = int(toks[3])
        pos += 1
        ch = 3 if magic == b"P6" else 1
        dt = np.uint8 if maxv < 256 else ">u2"
        arr = np.frombuffer(raw, dtype=dt, count=w * h * ch, offset=pos).reshape(h, w, ch).astype(np.float32)
        return torch.from_numpy(arr).permute(2, 0, 1)

    def load(self, path):
        ext = path.rsplit(".", 1)[-1].lower()
        if ext == "npy":
            t = torch.from_numpy(np.load(path)).float()
            t = t if t.dim() == 3 else t.unsqueeze(0)
        elif ext in ("ppm", "pgm", "pnm"):
            t = self._read_pnm(open(path, "rb").read())
        else:
            try:
                from PIL import Image
            except ImportError as e:
                raise IOError(f"decoding .{ext} images needs Pillow, which is not installed; convert to PPM/PGM or .npy") from e
            img = Image.open(path).convert("RGB" if self.c == 3 else "L")
            t = torch.from_numpy(np.asarray(img, dtype=np.float32))
            t = t.permute(2, 0, 1) if t.dim() == 3 else t.unsqueeze(0)
        if t.shape[0] != self.c:
            t = t.mean(0, keepdim=True) if self.c == 1 else t.expand(self.c, -1, -1)
        if t.shape[1:] != (self.h, self.w):
            t = torch.nn.functional.interpolate(t.unsqueeze(0), size=(self.h, self.w), mode="bilinear", align_corners=False).squeeze(0)
        return t

    def next(self):
        p = self._files[self._i]
        self._i += 1
        rec = [self.load(p)]
        if self.labelGen is not None:
            rec.append(self.labels.index(self.labelGen.getLabelForPath(p)))
        return rec


class TransformProcessRecordReader(RecordReader):
    def __init__(self, reader, transformProcess): self.reader, self.tp = reader, transformProcess
    def initialize(self, split, conf=None):
        self.reader.initialize(split, conf)
        self.reset()
        return self
    def reset(self):
        self.reader.reset()
        self._peek = self._pull()
    def _pull(self):
        while self.reader.hasNext():
            out = self.tp.execute(self.reader.next())
            if out is not None:
                return out
        return None
    def hasNext(self): return self._peek is not None
    def next(self):
        v = self._peek
        self._peek = self._pull()
        return v


class ConcatenatingRecordReader(RecordReader):
    def __init__(self, *readers): self.readers = list(readers)
    def initialize(self, split=None, conf=None):
        self.reset()
        return self
    def reset(self):
        for r in self.readers:
            r.reset()
        self._k = 0
    def hasNext(self):
        while self._k < len(self.readers) and not self.readers[self._k].hasNext():
            self._k += 1
        return self._k < len(self.readers)
    def next(self):
        self.hasNext()
        return self.readers[self._k].next()


class ComposableRecordReader(RecordReader):
    """Concatenates the columns of several readers stepping in lock-step."""
    def __init__(self, *readers): self.readers = list(readers)
    def initialize(self, split=None, conf=None):
        self.reset()
        return self
    def reset(self):
        for r in self.readers:
            r.reset()
    def hasNext(self): return all(r.hasNext() for r in self.readers)
    def next(self): return [v for r in self.readers for v in r.next()]


# ----------------------------------------------------------------------------- record writers
class CSVRecordWriter:
    def __init__(self, path, delimiter=","):
        self.f, self.delim = open(path, "w", newline=""), delimiter
    def write(self, record):
        self.f.write(self.delim.join(str(unwrap(v)) for v in record) + "\n")
    def writeBatch(self, records):
        for r in records:
            self.write(r)
    def close(self): self.f.close()


# ----------------------------------------------------------------------------- DataSet iterators over record readers
def _pin(t):
    return t.pin_memory() if torch.cuda.is_available() and not t.is_pinned() else t


class RecordReaderDataSetIterator:
    """Batches records into DataSets.  ``labelIndex`` (to ``labelIndexTo`` for multi-column regression) selects the label
    column(s); classification labels become one-hot rows of ``numPossibleLabels``; tensors in a record are concatenated
    (flattened) into the feature row unless the record is a single image tensor."""

    def __init__(self, recordReader, batchSize, labelIndex=-1, numPossibleLabels=-1, labelIndexTo=None, regression=False,
                 maxNumBatches=-1, preProcessor=None, collectMetaData=False):
        self.rr, self.batchSize, self.labelIndex, self.numLabels = recordReader, int(batchSize), labelIndex, numPossibleLabels
        self.labelIndexTo = labelIndex if labelIndexTo is None else labelIndexTo
        self.regression, self.maxNumBatches, self.preProcessor = regression, maxNumBatches, preProcessor
        self._batches = 0

    class Builder:
        def __init__(self, rr, batchSize): self.rr, self.kw = rr, {"batchSize": batchSize}
        def classification(self, labelIndex, numClasses): self.kw.update(labelIndex=labelIndex, numPossibleLabels=numClasses); return self
        def regression(self, frm, to=None): self.kw.update(labelIndex=frm, labelIndexTo=frm if to is None else to, regression=True); return self
        def maxNumBatches(self, n): self.kw["maxNumBatches"] = n; return self
        def preProcessor(self, p): self.kw["preProcessor"] = p; return self
        def collectMetaData(self, b): return self
        def build(self): return RecordReaderDataSetIterator(self.rr, **self.kw)

    def setPreProcessor(self, p): self.preProcessor = p
    def getPreProcessor(self): return self.preProcessor
    def getLabels(self): return self.rr.getLabels()
    def reset(self):
        self.rr.reset()
        self._batches = 0
    def resetSupported(self): return self.rr.resetSupported()
    def asyncSupported(self): return True
    def batch(self): return self.batchSize
    def hasNext(self): return self.rr.hasNext() and (self.maxNumBatches < 0 or self._batches < self.maxNumBatches)
    def inputColumns(self): return getattr(self, "_in_cols", None)
    def totalOutcomes(self): return self.numLabels

    def __iter__(self):
        self.reset()
        while self.hasNext():
            yield self.next()

    def next(self, n=None):
        recs = self.rr.nextBatch(n or self.batchSize)
        self._batches += 1
        li, lt = self.labelIndex, self.labelIndexTo
        if li is not None and li < 0 and self.numLabels > 0:
            li = lt = len(recs[0]) - 1
        feats, labs = [], []
        for r in recs:
            r = [unwrap(v) for v in r]
            if li is not None and li >= 0:
                lab = r[li:lt + 1]
                r = r[:li] + r[lt + 1:]
                labs.append(lab)
            if len(r) == 1 and isinstance(r[0], torch.Tensor):
                feats.append(r[0].float())
            else:
                parts = [v.reshape(-1).float() if isinstance(v, torch.Tensor) else torch.tensor([float(v)]) for v in r]
                feats.append(torch.cat(parts))
        x = _pin(torch.stack(feats))
        self._in_cols = x.shape[1] if x.dim() == 2 else None
        y = None
        if labs:
            if self.regression:
                y = torch.tensor([[float(v) for v in l] for l in labs], dtype=torch.float32)
            else:
                idx = torch.tensor([int(float(l[0])) for l in labs], dtype=torch.long)
                if self.numLabels <= 0:
                    raise ValueError("numPossibleLabels must be set for classification")
                y = torch.nn.functional.one_hot(idx, self.numLabels).float()
            y = _pin(y)
        ds = DataSet(x, y)
        if self.preProcessor is not None:
            self.preProcessor.preProcess(ds)
        return ds

    __next__ = next


class AlignmentMode:
    EQUAL_LENGTH = "EQUAL_LENGTH"
    ALIGN_START = "ALIGN_START"
    ALIGN_END = "ALIGN_END"


class SequenceRecordReaderDataSetIterator:
    """Sequences -> [N, C, T] DataSets with masks.  Either one reader (label column inside each step) or separate
    feature / label readers; ragged sequences are padded and aligned at the start or the end."""

    def __init__(self, featuresReader, *args, regression=False, alignmentMode=AlignmentMode.ALIGN_START):
        if args and hasattr(args[0], "hasNext"):
            # (featuresReader, labelsReader, miniBatchSize, numPossibleLabels[, regression[, alignmentMode]])
            self.fr, self.lr, self.batchSize = featuresReader, args[0], int(args[1])
            self.numLabels, self.labelIndex = (args[2] if len(args) > 2 else -1), None
            rest = args[3:]
        else:
            # (reader, miniBatchSize, numPossibleLabels, labelIndex[, regression])
            self.fr, self.lr, self.batchSize = featuresReader, None, int(args[0])
            self.numLabels, self.labelIndex = args[1], (args[2] if len(args) > 2 else -1)
            rest = args[3:]
        if rest:
            regression = bool(rest[0])
        if len(rest) > 1:
            alignmentMode = rest[1]
        self.regression, self.alignmentMode = regression, alignmentMode
        self.preProcessor = None

    def setPreProcessor(self, p): self.preProcessor = p
    def reset(self):
        self.fr.reset()
        if self.lr is not None:
            self.lr.reset()
    def resetSupported(self): return True
    def asyncSupported(self): return True
    def hasNext(self): return self.fr.hasNext()
    def __iter__(self):
        self.reset()
        while self.hasNext():
            yield self.next()

    def _labels(self, steps):
        if self.regression:
            return torch.tensor([[float(unwrap(v)) for v in s] for s in steps], dtype=torch.float32)
        idx = torch.tensor([int(float(unwrap(s[0]))) for s in steps], dtype=torch.long)
        return torch.nn.functional.one_hot(idx, self.numLabels).float()

    def next(self, n=None):
        fs, ls = [], []
        while self.fr.hasNext() and len(fs) < (n or self.batchSize):
            seq = self.fr.next()
            if self.lr is not None:
                lab = self.lr.next()
                fs.append(torch.tensor([[float(unwrap(v)) for v in s] for s in seq], dtype=torch.float32))
                ls.append(self._labels(lab))
            else:
                li = self.labelIndex if self.labelIndex >= 0 else len(seq[0]) - 1
                fs.append(torch.tensor([[float(unwrap(v)) for k, v in enumerate(s) if k != li] for s in seq], dtype=torch.float32))
                ls.append(self._labels([[s[li]] for s in seq]))
        T = max(max(f.shape[0] for f in fs), max(l.shape[0] for l in ls))
        N = len(fs)
        x = torch.zeros(N, fs[0].shape[1], T)
        y = torch.zeros(N, ls[0].shape[1], T)
        fm, lm = torch.zeros(N, T), torch.zeros(N, T)
        ragged = any(f.shape[0] != T for f in fs) or any(l.shape[0] != T for l in ls)
        if ragged and self.alignmentMode == AlignmentMode.EQUAL_LENGTH:
            raise ValueError("sequences differ in length: use AlignmentMode.ALIGN_START or ALIGN_END")
        for i, (f, l) in enumerate(zip(fs, ls)):
            for src, dst, msk in ((f, x, fm), (l, y, lm)):
                t = src.shape[0]
                o = T - t if self.alignmentMode == AlignmentMode.ALIGN_END else 0
                dst[i, :, o:o + t] = src.t()
                msk[i, o:o + t] = 1.0
        ds = DataSet(_pin(x), _pin(y), fm if ragged else None, lm if ragged else None)
        if self.preProcessor is not None:
            self.preProcessor.preProcess(ds)
        return ds

    __next__ = next
