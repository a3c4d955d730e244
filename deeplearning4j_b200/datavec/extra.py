"""DataVec pieces beyond the core record readers and ``TransformProcess``: joins, sequence operations, data-quality analysis,
Arrow / JDBC / Excel record readers and writers, the image loader and image transforms.

Reference packages: ``datavec-api/.../transform/join/Join.java``, ``transform/sequence/**`` (trim, window reduce, difference,
split), ``transform/quality/**`` + ``datavec-local/.../AnalyzeLocal.java``, ``datavec-arrow/.../ArrowConverter.java`` and
``ArrowRecordReader.java``, ``datavec-jdbc/.../JDBCRecordReader.java``, ``datavec-excel/.../ExcelRecordReader.java``,
``datavec-data-image/.../NativeImageLoader.java`` and ``transform/*ImageTransform.java``.
"""
from __future__ import annotations

import math
import os
import re
import zipfile
from collections import OrderedDict
from xml.etree import ElementTree as ET
from xml.sax.saxutils import escape

import numpy as np
import torch

from .records import RecordReader, Writable, unwrap
from .transform import ColumnMeta, ColumnType, Schema, _reduce


# ====================================================================================================== joins
class JoinType:
    Inner, LeftOuter, RightOuter, FullOuter = "Inner", "LeftOuter", "RightOuter", "FullOuter"


class Join:
    """Key-based join of two record collections.  The output columns are the left schema followed by the right schema without
    its key columns; rows without a partner are padded with ``None`` on the outer sides."""

    def __init__(self, joinType, leftSchema, rightSchema, keysLeft, keysRight):
        self.joinType, self.left, self.right = joinType, leftSchema, rightSchema
        self.keysLeft, self.keysRight = list(keysLeft), list(keysRight)
        if len(self.keysLeft) != len(self.keysRight) or not self.keysLeft:
            raise ValueError("join needs the same (non-zero) number of key columns on both sides")
        for k in self.keysLeft:
            leftSchema.getIndexOfColumn(k)
        for k in self.keysRight:
            rightSchema.getIndexOfColumn(k)

    class Builder:
        def __init__(self, joinType): self.joinType, self.l, self.r, self.kl, self.kr = joinType, None, None, None, None
        def setSchemas(self, left, right): self.l, self.r = left, right; return self
        def setJoinColumns(self, *c): self.kl = self.kr = list(c); return self
        setKeyColumns = setJoinColumns
        def setJoinColumnsLeft(self, *c): self.kl = list(c); return self
        def setJoinColumnsRight(self, *c): self.kr = list(c); return self
        setKeyColumnsLeft, setKeyColumnsRight = setJoinColumnsLeft, setJoinColumnsRight
        def build(self): return Join(self.joinType, self.l, self.r, self.kl, self.kr)

    def getOutputSchema(self):
        cols = list(self.left.columns) + [c for c in self.right.columns if c.name not in self.keysRight]
        names = [c.name for c in cols]
        if len(set(names)) != len(names):
            raise ValueError(f"join would produce duplicate column names: {names}")
        return Schema(cols)

    def execute(self, leftRecords, rightRecords):
        li = [self.left.getIndexOfColumn(k) for k in self.keysLeft]
        ri = [self.right.getIndexOfColumn(k) for k in self.keysRight]
        rest = [i for i in range(len(self.right.columns)) if i not in ri]
        nl = len(self.left.columns)
        index = OrderedDict()
        for r in rightRecords:
            index.setdefault(tuple(unwrap(r[i]) for i in ri), []).append(list(r))
        used, out = set(), []
        for l in leftRecords:
            key = tuple(unwrap(l[i]) for i in li)
            partners = index.get(key)
            if partners:
                used.add(key)
                for r in partners:
                    out.append(list(l) + [r[i] for i in rest])
            elif self.joinType in (JoinType.LeftOuter, JoinType.FullOuter):
                out.append(list(l) + [None] * len(rest))
        if self.joinType in (JoinType.RightOuter, JoinType.FullOuter):
            for key, partners in index.items():
                if key in used:
                    continue
                for r in partners:
                    row = [None] * nl
                    for a, b in zip(li, ri):
                        row[a] = r[b]
                    out.append(row + [r[i] for i in rest])
        return out


def executeJoin(join, left, right):
    """``LocalTransformExecutor.executeJoin``."""
    return join.execute(left, right)


# ====================================================================================================== sequence operations
def _col(schema, name): return schema.getIndexOfColumn(name)


def trimSequence(sequences, numSteps, fromFirst=True):
    """``SequenceTrimTransform``: drop ``numSteps`` steps from the start (or the end) of every sequence."""
    return [s[numSteps:] if fromFirst else s[:max(len(s) - numSteps, 0)] for s in sequences]


def trimSequenceToLength(sequences, maxLength, pad=False, padValue=None):
    """``SequenceTrimToLengthTransform``: cut to ``maxLength`` steps; with ``pad`` shorter sequences are extended with ``padValue`` rows."""
    out = []
    for s in sequences:
        s = list(s[:maxLength])
        if pad and len(s) < maxLength and s:
            s += [list(padValue) if padValue is not None else list(s[-1]) for _ in range(maxLength - len(s))]
        out.append(s)
    return out


def sequenceDifference(schema, sequences, column, lookback=1, firstStep="Default", specified=None):
    """``SequenceDifferenceTransform``: x[t] - x[t - lookback]; the first ``lookback`` steps give 0 (``Default``) or ``specified``."""
    i = _col(schema, column)
    out = []
    for s in sequences:
        new = []
        for t, row in enumerate(s):
            row = list(row)
            if t < lookback:
                row[i] = 0 if firstStep == "Default" else specified
            else:
                row[i] = unwrap(s[t][i]) - unwrap(s[t - lookback][i])
            new.append(row)
        out.append(new)
    return out


def sequenceMovingWindowReduce(schema, sequences, column, lookback, op, edge="Default"):
    """``SequenceMovingWindowReduceTransform``: appends ``<op>(<lookback>,<column>)`` holding the reduction of the last
    ``lookback`` values (fewer at the start; ``edge='SpecifiedValue'`` writes None there instead)."""
    i = _col(schema, column)
    out = []
    for s in sequences:
        new = []
        for t, row in enumerate(s):
            lo = max(0, t - lookback + 1)
            if edge != "Default" and t - lookback + 1 < 0:
                v = None
            else:
                v = _reduce(op, [unwrap(r[i]) for r in s[lo:t + 1]])
            new.append(list(row) + [v])
        out.append(new)
    t = ColumnType.Long if op in ("Count", "CountUnique") else ColumnType.Double
    return out, Schema(list(schema.columns) + [ColumnMeta(f"{op.lower()}({lookback},{column})", t)])


def reduceSequence(schema, sequences, reducer):
    """``ReduceSequenceTransform``: every sequence becomes one record through a ``Reducer`` (its key columns are ignored)."""
    rows = []
    for s in sequences:
        row = []
        for i, c in enumerate(schema.columns):
            row.append(_reduce(reducer.ops.get(c.name, reducer.defaultOp), [unwrap(r[i]) for r in s]))
        rows.append(row)
    return rows


def convertFromSequence(sequences):
    """Flatten sequences back into independent records."""
    return [list(r) for s in sequences for r in s]


def splitSequenceMaxLength(sequences, maxLength, equalSplits=False):
    """``SplitMaxLengthSequence``: sequences longer than ``maxLength`` are cut into pieces (of equal length when asked)."""
    out = []
    for s in sequences:
        if len(s) <= maxLength:
            out.append(list(s))
            continue
        if equalSplits:
            n = math.ceil(len(s) / maxLength)
            size = math.ceil(len(s) / n)
        else:
            size = maxLength
        out += [list(s[k:k + size]) for k in range(0, len(s), size)]
    return out


def splitSequenceTimeSeparation(schema, sequences, timeColumn, maxGap):
    """``SequenceSplitTimeSeparation``: a new sequence starts wherever two consecutive time stamps are more than ``maxGap`` apart."""
    i = _col(schema, timeColumn)
    out = []
    for s in sequences:
        cur = []
        for row in s:
            if cur and unwrap(row[i]) - unwrap(cur[-1][i]) > maxGap:
                out.append(cur)
                cur = []
            cur.append(list(row))
        if cur:
            out.append(cur)
    return out


# ====================================================================================================== data quality
class ColumnQuality:
    def __init__(self, **kw): self.__dict__.update(kw)
    def __repr__(self): return ", ".join(f"{k}={v}" for k, v in self.__dict__.items())


class DataQualityAnalysis:
    def __init__(self, schema, columns): self.schema, self.columns = schema, columns
    def getColumnQualityList(self): return [self.columns[c.name] for c in self.schema.columns]
    def getColumnQuality(self, name): return self.columns[name]
    def __repr__(self): return "\n".join(f"{k}: {v}" for k, v in self.columns.items())


def analyzeQuality(schema, records):
    """``AnalyzeLocal.analyzeQuality``: per column the number of valid, invalid, missing (None / empty) and total values, plus
    type-specific counts (non-integer / NaN / infinite for numeric columns, empty / unique for strings, unknown states for
    categorical columns)."""
    cols = {}
    for i, c in enumerate(schema.columns):
        vals = [unwrap(r[i]) if i < len(r) else None for r in records]
        q = dict(countValid=0, countInvalid=0, countMissing=0, countTotal=len(vals))
        numeric = c.type in (ColumnType.Integer, ColumnType.Long, ColumnType.Double, ColumnType.Float, ColumnType.Time)
        if numeric:
            q.update(countNonNumeric=0, countNaN=0, countInfinite=0)
            if c.type in (ColumnType.Integer, ColumnType.Long, ColumnType.Time):
                q["countNonInteger"] = 0
        elif c.type == ColumnType.String:
            q.update(countEmptyString=0, countUnique=0)
        states = set(c.extra.get("stateNames") or [])
        seen = set()
        for v in vals:
            if v is None or (isinstance(v, str) and v == "" and c.type != ColumnType.String):
                q["countMissing"] += 1
                continue
            if numeric:
                try:
                    f = float(v)
                except (TypeError, ValueError):
                    q["countNonNumeric"] += 1
                    q["countInvalid"] += 1
                    continue
                if math.isnan(f):
                    q["countNaN"] += 1
                    q["countInvalid"] += 1
                elif math.isinf(f):
                    q["countInfinite"] += 1
                    q["countInvalid"] += 1
                elif "countNonInteger" in q and (isinstance(v, str) and not re.fullmatch(r"[+-]?\d+", v.strip()) or f != int(f)):
                    q["countNonInteger"] += 1
                    q["countInvalid"] += 1
                else:
                    q["countValid"] += 1
            elif c.type == ColumnType.String:
                seen.add(v)
                if v == "":
                    q["countEmptyString"] += 1
                q["countValid"] += 1
            elif c.type == ColumnType.Categorical and states:
                if str(v) in states:
                    q["countValid"] += 1
                else:
                    q["countInvalid"] += 1
            else:
                q["countValid"] += 1
        if c.type == ColumnType.String:
            q["countUnique"] = len(seen)
        cols[c.name] = ColumnQuality(**q)
    return DataQualityAnalysis(schema, cols)


# ====================================================================================================== Arrow
_ARROW_TYPES = None


def _arrow_type(t):
    import pyarrow as pa
    return {ColumnType.Integer: pa.int32(), ColumnType.Long: pa.int64(), ColumnType.Double: pa.float64(), ColumnType.Float: pa.float32(),
            ColumnType.Time: pa.int64(), ColumnType.Boolean: pa.bool_()}.get(t, pa.string())


class ArrowConverter:
    """Records <-> Arrow record batches / IPC files (``ArrowConverter.toArrowColumns`` / ``writeRecordBatchTo`` / ``readFromFile``)."""

    @staticmethod
    def toArrowTable(schema, records):
        import pyarrow as pa
        cols = []
        for i, c in enumerate(schema.columns):
            vals = [unwrap(r[i]) for r in records]
            at = _arrow_type(c.type)
            if pa.types.is_string(at):
                vals = [None if v is None else str(v) for v in vals]
            cols.append(pa.array(vals, type=at))
        return pa.table(cols, names=[c.name for c in schema.columns])

    @staticmethod
    def toSchema(arrowSchema):
        import pyarrow as pa
        cols = []
        for f in arrowSchema:
            t = (ColumnType.Integer if pa.types.is_int32(f.type) or pa.types.is_int16(f.type) or pa.types.is_int8(f.type) else
                 ColumnType.Long if pa.types.is_integer(f.type) else
                 ColumnType.Float if pa.types.is_float32(f.type) else
                 ColumnType.Double if pa.types.is_floating(f.type) else
                 ColumnType.Boolean if pa.types.is_boolean(f.type) else ColumnType.String)
            cols.append(ColumnMeta(f.name, t))
        return Schema(cols)

    @staticmethod
    def toRecords(table):
        cols = [c.to_pylist() for c in table.columns]
        return [list(r) for r in zip(*cols)] if cols else []

    @staticmethod
    def writeRecordBatchTo(records, schema, path):
        import pyarrow as pa
        t = ArrowConverter.toArrowTable(schema, records)
        with pa.OSFile(path, "wb") as sink, pa.ipc.new_file(sink, t.schema) as w:
            w.write_table(t)

    @staticmethod
    def readFromFile(path):
        import pyarrow as pa
        with pa.memory_map(path, "r") as src:
            t = pa.ipc.open_file(src).read_all()
        return ArrowConverter.toSchema(t.schema), ArrowConverter.toRecords(t)

    @staticmethod
    def toTensor(table, dtype=torch.float32):
        """Numeric columns of a table as one [rows, columns] tensor without a Python loop over rows."""
        return torch.from_numpy(np.stack([np.asarray(c.to_numpy(zero_copy_only=False), dtype=np.float64) for c in table.columns], 1)).to(dtype)


class ArrowRecordReader(RecordReader):
    """Reads Arrow IPC files (one or several) record by record."""

    def reset(self):
        self._rows = []
        for p in self.split.locations():
            self.schema, rows = ArrowConverter.readFromFile(p)
            self._rows += rows
        self._i = 0

    def hasNext(self): return self._i < len(self._rows)

    def next(self):
        r = self._rows[self._i]
        self._i += 1
        return list(r)


class ArrowRecordWriter:
    def __init__(self, schema, path): self.schema, self.path, self._rows = schema, path, []
    def write(self, record): self._rows.append(list(record))
    def writeBatch(self, records): self._rows += [list(r) for r in records]
    def close(self): ArrowConverter.writeRecordBatchTo(self._rows, self.schema, self.path)


# ====================================================================================================== JDBC
class JDBCRecordReader(RecordReader):
    """Rows of an SQL query as records, over any DB-API 2.0 connection (``sqlite3`` ships with Python; the reference wraps a
    ``javax.sql.DataSource``).  ``metaDataQuery`` + ``metaDataIndices``, when given, produce the record's key for ``loadFromMetaData``."""

    def __init__(self, query, connection=None, connectionFactory=None, metaDataQuery=None, metaDataIndices=None):
        self.query, self.conn, self.factory = query, connection, connectionFactory
        self.metaDataQuery, self.metaDataIndices = metaDataQuery, metaDataIndices
        self._cur = None

    def initialize(self, split=None):
        if self.conn is None:
            if self.factory is None:
                raise ValueError("JDBCRecordReader needs a connection or a connection factory")
            self.conn = self.factory()
        self.reset()
        return self

    def reset(self):
        self._cur = self.conn.cursor()
        self._cur.execute(self.query)
        self.labels = [d[0] for d in self._cur.description]
        self._next = self._cur.fetchone()

    def getLabels(self): return self.labels
    def hasNext(self): return self._next is not None

    def next(self):
        r = list(self._next)
        self._next = self._cur.fetchone()
        return r

    def nextRecordWithMeta(self):
        r = self.next()
        meta = [r[i] for i in (self.metaDataIndices or [])]
        return r, meta

    def loadFromMetaData(self, meta):
        if not self.metaDataQuery:
            raise ValueError("no metaDataQuery was set")
        cur = self.conn.cursor()
        cur.execute(self.metaDataQuery, tuple(meta))
        row = cur.fetchone()
        return None if row is None else list(row)

    def close(self):
        if self._cur is not None:
            self._cur.close()


# ====================================================================================================== Excel (.xlsx)
_NS = {"m": "http://schemas.openxmlformats.org/spreadsheetml/2006/main"}


def _col_index(ref):
    n = 0
    for ch in re.match(r"[A-Z]+", ref).group(0):
        n = n * 26 + ord(ch) - 64
    return n - 1


def _col_name(i):
    s = ""
    i += 1
    while i:
        i, r = divmod(i - 1, 26)
        s = chr(65 + r) + s
    return s


class ExcelRecordReader(RecordReader):
    """Rows of the sheets of ``.xlsx`` workbooks (the zipped SpreadsheetML parts are parsed directly: shared and inline strings,
    numbers, booleans).  ``skipNumLines`` header rows are skipped per sheet."""

    def __init__(self, skipNumLines=0): self.skip = skipNumLines

    @staticmethod
    def _sheet_rows(z, name, shared):
        rows = []
        root = ET.fromstring(z.read(name))
        for row in root.iterfind(".//m:sheetData/m:row", _NS):
            vals = []
            for c in row.iterfind("m:c", _NS):
                i = _col_index(c.get("r")) if c.get("r") else len(vals)
                while len(vals) < i:
                    vals.append(None)
                t, v = c.get("t", "n"), c.find("m:v", _NS)
                if t == "s":
                    vals.append(shared[int(v.text)])
                elif t == "inlineStr":
                    vals.append("".join(x.text or "" for x in c.iterfind(".//m:t", _NS)))
                elif t == "b":
                    vals.append(v.text == "1")
                elif t == "str":
                    vals.append(v.text if v is not None else "")
                elif v is None or v.text is None:
                    vals.append(None)
                else:
                    f = float(v.text)
                    vals.append(int(f) if f == int(f) and "." not in v.text and "E" not in v.text.upper() else f)
            rows.append(vals)
        return rows

    def reset(self):
        self._rows = []
        for p in self.split.locations():
            with zipfile.ZipFile(p) as z:
                shared = []
                if "xl/sharedStrings.xml" in z.namelist():
                    for si in ET.fromstring(z.read("xl/sharedStrings.xml")).iterfind("m:si", _NS):
                        shared.append("".join(x.text or "" for x in si.iterfind(".//m:t", _NS)))
                sheets = sorted((n for n in z.namelist() if re.fullmatch(r"xl/worksheets/sheet\d+\.xml", n)),
                                key=lambda n: int(re.search(r"\d+", n.rsplit("/", 1)[1]).group(0)))
                for s in sheets:
                    self._rows += self._sheet_rows(z, s, shared)[self.skip:]
        self._i = 0

    def hasNext(self): return self._i < len(self._rows)

    def next(self):
        r = self._rows[self._i]
        self._i += 1
        return list(r)


class ExcelRecordWriter:
    """Writes records as the single sheet of a minimal ``.xlsx`` workbook (inline strings)."""

    def __init__(self, path, sheetName="Sheet1"): self.path, self.sheet, self._rows = path, sheetName, []
    def write(self, record): self._rows.append([unwrap(v) for v in record])
    def writeBatch(self, records): [self.write(r) for r in records]

    def close(self):
        body = []
        for ri, row in enumerate(self._rows, 1):
            cells = []
            for ci, v in enumerate(row):
                ref = f"{_col_name(ci)}{ri}"
                if v is None:
                    continue
                if isinstance(v, bool):
                    cells.append(f'<c r="{ref}" t="b"><v>{int(v)}</v></c>')
                elif isinstance(v, (int, float)):
                    cells.append(f'<c r="{ref}"><v>{v!r}</v></c>')
                else:
                    cells.append(f'<c r="{ref}" t="inlineStr"><is><t>{escape(str(v))}</t></is></c>')
            body.append(f'<row r="{ri}">{"".join(cells)}</row>')
        main = "http://schemas.openxmlformats.org/spreadsheetml/2006/main"
        rel = "http://schemas.openxmlformats.org/officeDocument/2006/relationships"
        with zipfile.ZipFile(self.path, "w", zipfile.ZIP_DEFLATED) as z:
            z.writestr("[Content_Types].xml",
                       '<?xml version="1.0" encoding="UTF-8"?><Types xmlns="http://schemas.openxmlformats.org/package/2006/content-types">'
                       '<Default Extension="rels" ContentType="application/vnd.openxmlformats-package.relationships+xml"/>'
                       '<Default Extension="xml" ContentType="application/xml"/>'
                       '<Override PartName="/xl/workbook.xml" ContentType="application/vnd.openxmlformats-officedocument.spreadsheetml.sheet.main+xml"/>'
                       '<Override PartName="/xl/worksheets/sheet1.xml" ContentType="application/vnd.openxmlformats-officedocument.spreadsheetml.worksheet+xml"/>'
                       '</Types>')
            z.writestr("_rels/.rels", f'<?xml version="1.0" encoding="UTF-8"?><Relationships xmlns="http://schemas.openxmlformats.org/package/2006/relationships">'
                       f'<Relationship Id="rId1" Type="{rel}/officeDocument" Target="xl/workbook.xml"/></Relationships>')
            z.writestr("xl/workbook.xml", f'<?xml version="1.0" encoding="UTF-8"?><workbook xmlns="{main}" xmlns:r="{rel}"><sheets>'
                       f'<sheet name="{escape(self.sheet)}" sheetId="1" r:id="rId1"/></sheets></workbook>')
            z.writestr("xl/_rels/workbook.xml.rels", f'<?xml version="1.0" encoding="UTF-8"?><Relationships xmlns="http://schemas.openxmlformats.org/package/2006/relationships">'
                       f'<Relationship Id="rId1" Type="{rel}/worksheet" Target="worksheets/sheet1.xml"/></Relationships>')
            z.writestr("xl/worksheets/sheet1.xml", f'<?xml version="1.0" encoding="UTF-8"?><worksheet xmlns="{main}"><sheetData>{"".join(body)}</sheetData></worksheet>')


# ====================================================================================================== images
class NativeImageLoader:
    """Image file / array -> ``[1, C, H, W]`` float tensor, resized to (height, width) and converted to ``channels``
    (``NativeImageLoader.asMatrix``); ``asRowVector`` flattens it."""

    ALLOWED_FORMATS = ("bmp", "gif", "jpg", "jpeg", "jp2", "pbm", "pgm", "ppm", "pnm", "png", "tif", "tiff", "npy")

    def __init__(self, height=-1, width=-1, channels=-1, centerCropIfNeeded=False, imageTransform=None):
        self.h, self.w, self.c, self.centerCrop, self.transform = height, width, channels, centerCropIfNeeded, imageTransform

    def _decode(self, src):
        if isinstance(src, torch.Tensor):
            return src.float() if src.dim() == 3 else src.float().unsqueeze(0)
        if isinstance(src, np.ndarray):
            t = torch.from_numpy(np.ascontiguousarray(src)).float()
            return t.permute(2, 0, 1) if t.dim() == 3 else t.unsqueeze(0)
        path = os.fspath(src)
        if path.lower().endswith(".npy"):
            return self._decode(torch.from_numpy(np.load(path)))
        from PIL import Image
        img = Image.open(path)
        if img.mode not in ("L", "RGB", "RGBA"):
            img = img.convert("RGB")
        return self._decode(np.asarray(img, dtype=np.float32))

    def asMatrix(self, src):
        t = self._decode(src)
        if self.transform is not None:
            t = self.transform.transform(t)
        if self.c > 0 and t.shape[0] != self.c:
            if self.c == 1:
                t = (0.299 * t[0] + 0.587 * t[1] + 0.114 * t[2]).unsqueeze(0) if t.shape[0] >= 3 else t[:1]
            elif t.shape[0] == 1:
                t = t.expand(self.c, -1, -1)
            else:
                t = t[:self.c] if t.shape[0] > self.c else torch.cat([t, torch.full((self.c - t.shape[0], *t.shape[1:]), 255.0)])
        if self.h > 0 and self.w > 0 and tuple(t.shape[1:]) != (self.h, self.w):
            if self.centerCrop:
                H, W = t.shape[1:]
                ar = self.w / self.h
                ch, cw = (H, int(round(H * ar))) if W / H > ar else (int(round(W / ar)), W)
                t = t[:, (H - ch) // 2:(H - ch) // 2 + ch, (W - cw) // 2:(W - cw) // 2 + cw]
            t = torch.nn.functional.interpolate(t.unsqueeze(0), size=(self.h, self.w), mode="bilinear", align_corners=False).squeeze(0)
        return t.unsqueeze(0).contiguous()

    def asRowVector(self, src): return self.asMatrix(src).reshape(1, -1)
    def asImageMatrix(self, src): return self.asMatrix(src)

    @staticmethod
    def asFile(tensor, path):
        """Writes a ``[C, H, W]`` (or ``[1, C, H, W]``) tensor with values in 0..255 as an image file."""
        from PIL import Image
        t = tensor[0] if tensor.dim() == 4 else tensor
        a = t.clamp(0, 255).to(torch.uint8).permute(1, 2, 0).cpu().numpy()
        Image.fromarray(a[:, :, 0] if a.shape[2] == 1 else a).save(path)


class ImageTransform:
    def transform(self, t, rng=None): raise NotImplementedError
    def __call__(self, t): return self.transform(t)


class _Rand:
    def __init__(self, seed): self.g = torch.Generator().manual_seed(int(seed) if seed is not None else 0)
    def uniform(self, lo, hi): return lo + (hi - lo) * float(torch.rand((), generator=self.g))
    def randint(self, lo, hi): return int(torch.randint(lo, hi + 1, (), generator=self.g))


class FlipImageTransform(ImageTransform):
    """flipMode 0: around the x axis (up-down), 1: around the y axis (left-right), -1: both; None: random choice per call."""
    def __init__(self, flipMode=None, seed=None): self.mode, self.r = flipMode, _Rand(seed)
    def transform(self, t, rng=None):
        m = self.mode if self.mode is not None else self.r.randint(-1, 1)
        return t.flip(1) if m == 0 else t.flip(2) if m == 1 else t.flip(1, 2)


class CropImageTransform(ImageTransform):
    """Removes up to (top, left, bottom, right) pixels; with a seed the amounts are drawn uniformly from [0, bound]."""
    def __init__(self, cropTop, cropLeft=None, cropBottom=None, cropRight=None, seed=None):
        cropLeft = cropTop if cropLeft is None else cropLeft
        self.b = (cropTop, cropLeft, cropTop if cropBottom is None else cropBottom, cropLeft if cropRight is None else cropRight)
        self.r = _Rand(seed) if seed is not None else None
    def transform(self, t, rng=None):
        tp, lf, bt, rt = (self.r.randint(0, v) for v in self.b) if self.r else self.b
        return t[:, tp:t.shape[1] - bt, lf:t.shape[2] - rt]


class RandomCropTransform(ImageTransform):
    def __init__(self, height, width, seed=None): self.h, self.w, self.r = height, width, _Rand(seed)
    def transform(self, t, rng=None):
        y, x = self.r.randint(0, t.shape[1] - self.h), self.r.randint(0, t.shape[2] - self.w)
        return t[:, y:y + self.h, x:x + self.w]


class ResizeImageTransform(ImageTransform):
    def __init__(self, newWidth, newHeight): self.w, self.h = newWidth, newHeight
    def transform(self, t, rng=None):
        return torch.nn.functional.interpolate(t.unsqueeze(0), size=(self.h, self.w), mode="bilinear", align_corners=False).squeeze(0)


class ScaleImageTransform(ImageTransform):
    """Scales by a factor drawn from [1 - delta, 1 + delta] per axis (``delta`` in pixels when > 1, as in the reference)."""
    def __init__(self, dx, dy=None, seed=None): self.dx, self.dy, self.r = dx, dx if dy is None else dy, _Rand(seed)
    def transform(self, t, rng=None):
        H, W = t.shape[1:]
        nh = max(1, int(round(H + self.r.uniform(-self.dy, self.dy)))) if self.dy >= 1 else max(1, int(round(H * (1 + self.r.uniform(-self.dy, self.dy)))))
        nw = max(1, int(round(W + self.r.uniform(-self.dx, self.dx)))) if self.dx >= 1 else max(1, int(round(W * (1 + self.r.uniform(-self.dx, self.dx)))))
        return torch.nn.functional.interpolate(t.unsqueeze(0), size=(nh, nw), mode="bilinear", align_corners=False).squeeze(0)


class RotateImageTransform(ImageTransform):
    """Rotation about the centre by an angle (degrees) drawn from [-angle, angle]; the canvas keeps its size."""
    def __init__(self, angle, seed=None, fixed=False): self.a, self.r, self.fixed = angle, _Rand(seed), fixed
    def transform(self, t, rng=None):
        th = math.radians(self.a if self.fixed else self.r.uniform(-self.a, self.a))
        H, W = t.shape[1:]
        c, s = math.cos(th), math.sin(th)
        theta = torch.tensor([[c, -s * H / W, 0.0], [s * W / H, c, 0.0]], dtype=torch.float32).unsqueeze(0)
        grid = torch.nn.functional.affine_grid(theta, (1, t.shape[0], H, W), align_corners=False)
        return torch.nn.functional.grid_sample(t.unsqueeze(0).float(), grid, mode="bilinear", padding_mode="zeros", align_corners=False).squeeze(0)


class ColorConversionTransform(ImageTransform):
    """RGB -> grey ('GRAY'), RGB <-> BGR ('BGR'), RGB -> YCrCb ('YCrCb') or RGB -> HSV ('HSV', H in degrees / 2 like OpenCV's 8-bit form)."""
    def __init__(self, conversion="GRAY"): self.conv = conversion.upper()
    def transform(self, t, rng=None):
        r, g, b = t[0], t[1], t[2]
        if self.conv == "GRAY":
            return (0.299 * r + 0.587 * g + 0.114 * b).unsqueeze(0)
        if self.conv == "BGR":
            return t.flip(0)
        if self.conv == "YCRCB":
            y = 0.299 * r + 0.587 * g + 0.114 * b
            return torch.stack([y, (r - y) * 0.713 + 128.0, (b - y) * 0.564 + 128.0])
        if self.conv == "HSV":
            mx, mn = t.amax(0), t.amin(0)
            d = mx - mn
            h = torch.zeros_like(mx)
            nz = d > 0
            h = torch.where(nz & (mx == r), 60.0 * ((g - b) / d.clamp_min(1e-12)) % 360.0, h)
            h = torch.where(nz & (mx == g) & (mx != r), 60.0 * ((b - r) / d.clamp_min(1e-12)) + 120.0, h)
            h = torch.where(nz & (mx == b) & (mx != r) & (mx != g), 60.0 * ((r - g) / d.clamp_min(1e-12)) + 240.0, h)
            s = torch.where(mx > 0, d / mx.clamp_min(1e-12), torch.zeros_like(mx)) * 255.0
            return torch.stack([h / 2.0, s, mx])
        raise ValueError(f"unknown colour conversion {self.conv}")


class EqualizeHistTransform(ImageTransform):
    """Histogram equalisation of every channel (values 0..255)."""
    def transform(self, t, rng=None):
        out = []
        for ch in t:
            v = ch.clamp(0, 255).to(torch.int64).reshape(-1)
            hist = torch.bincount(v, minlength=256).double()
            cdf = hist.cumsum(0)
            lo = cdf[hist > 0][0]
            lut = ((cdf - lo) / max(float(cdf[-1] - lo), 1.0) * 255.0).round().clamp(0, 255)
            out.append(lut[v].reshape(ch.shape).float())
        return torch.stack(out)


class BoxImageTransform(ImageTransform):
    """Centres the image on a (width, height) canvas: crops what is larger, pads with ``borderValue`` what is smaller."""
    def __init__(self, width, height, borderValue=0.0): self.w, self.h, self.v = width, height, borderValue
    def transform(self, t, rng=None):
        C, H, W = t.shape
        out = torch.full((C, self.h, self.w), float(self.v))
        sy, sx = max((H - self.h) // 2, 0), max((W - self.w) // 2, 0)
        dy, dx = max((self.h - H) // 2, 0), max((self.w - W) // 2, 0)
        hh, ww = min(H, self.h), min(W, self.w)
        out[:, dy:dy + hh, dx:dx + ww] = t[:, sy:sy + hh, sx:sx + ww]
        return out


class PipelineImageTransform(ImageTransform):
    """Applies (transform, probability) pairs in order (optionally shuffled), each with its probability."""
    def __init__(self, transforms, shuffle=False, seed=None):
        self.items = [(t, 1.0) if isinstance(t, ImageTransform) else (t[0], float(t[1])) for t in transforms]
        self.shuffle, self.r = shuffle, _Rand(seed)
    def transform(self, t, rng=None):
        items = list(self.items)
        if self.shuffle:
            order = torch.randperm(len(items), generator=self.r.g).tolist()
            items = [items[i] for i in order]
        for tr, p in items:
            if p >= 1.0 or self.r.uniform(0.0, 1.0) < p:
                t = tr.transform(t)
        return t


class MultiImageTransform(PipelineImageTransform):
    def __init__(self, *transforms): super().__init__(list(transforms))
