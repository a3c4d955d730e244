"""``Schema`` and ``TransformProcess`` (``datavec-api/.../api/transform``): column metadata, the builder of
column operations (remove / rename / categorical <-> integer / one-hot, math ops, string ops, conditional
replace, filters, reducers, sequence conversion), a local executor and JSON serialisation."""
from __future__ import annotations

import json
import math
import re
from collections import OrderedDict

from .records import unwrap


class ColumnType:
    String = "String"
    Integer = "Integer"
    Long = "Long"
    Double = "Double"
    Float = "Float"
    Categorical = "Categorical"
    Time = "Time"
    Bytes = "Bytes"
    Boolean = "Boolean"
    NDArray = "NDArray"


class ColumnMeta:
    def __init__(self, name, ctype, **kw):
        self.name, self.type, self.extra = name, ctype, kw
    def to_dict(self): return {"name": self.name, "type": self.type, **self.extra}
    def __repr__(self): return f"{self.name}:{self.type}"


class Schema:
    def __init__(self, columns=()):
        self.columns = list(columns)

    class Builder:
        def __init__(self): self.cols = []
        def _add(self, t, names, **kw):
            for n in names:
                self.cols.append(ColumnMeta(n, t, **kw))
            return self
        def addColumnString(self, *n): return self._add(ColumnType.String, n)
        addColumnsString = addColumnString
        def addColumnInteger(self, *n, **kw): return self._add(ColumnType.Integer, n, **kw)
        addColumnsInteger = addColumnInteger
        def addColumnLong(self, *n): return self._add(ColumnType.Long, n)
        addColumnsLong = addColumnLong
        def addColumnDouble(self, *n, **kw): return self._add(ColumnType.Double, n, **kw)
        addColumnsDouble = addColumnDouble
        def addColumnFloat(self, *n): return self._add(ColumnType.Float, n)
        addColumnsFloat = addColumnFloat
        def addColumnBoolean(self, *n): return self._add(ColumnType.Boolean, n)
        def addColumnTime(self, name, timeZone="UTC"): return self._add(ColumnType.Time, [name], timeZone=timeZone)
        def addColumnNDArray(self, name, shape): return self._add(ColumnType.NDArray, [name], shape=list(shape))
        def addColumnCategorical(self, name, *states):
            states = list(states[0]) if len(states) == 1 and isinstance(states[0], (list, tuple)) else list(states)
            return self._add(ColumnType.Categorical, [name], stateNames=states)
        def build(self): return Schema(self.cols)

    def numColumns(self): return len(self.columns)
    def getColumnNames(self): return [c.name for c in self.columns]
    def getColumnTypes(self): return [c.type for c in self.columns]
    def getIndexOfColumn(self, name):
        for i, c in enumerate(self.columns):
            if c.name == name:
                return i
        raise KeyError(f"no column named {name!r}; columns: {self.getColumnNames()}")
    def hasColumn(self, name): return name in self.getColumnNames()
    def getName(self, i): return self.columns[i].name
    def getType(self, i): return self.columns[self.getIndexOfColumn(i)].type if isinstance(i, str) else self.columns[i].type
    def getMetaData(self, i): return self.columns[self.getIndexOfColumn(i)] if isinstance(i, str) else self.columns[i]
    def toJson(self): return json.dumps({"columns": [c.to_dict() for c in self.columns]})
    @staticmethod
    def fromJson(s): return Schema([ColumnMeta(d.pop("name"), d.pop("type"), **d) for d in json.loads(s)["columns"]])
    def __repr__(self): return "Schema(" + ", ".join(map(repr, self.columns)) + ")"
    def __eq__(self, o): return isinstance(o, Schema) and self.toJson() == o.toJson()


# ----------------------------------------------------------------------------- conditions
class ConditionOp:
    LessThan, LessOrEqual, GreaterThan, GreaterOrEqual, Equal, NotEqual, InSet, NotInSet = (
        "LessThan", "LessOrEqual", "GreaterThan", "GreaterOrEqual", "Equal", "NotEqual", "InSet", "NotInSet")


_OPS = {"LessThan": lambda a, b: a < b, "LessOrEqual": lambda a, b: a <= b, "GreaterThan": lambda a, b: a > b,
        "GreaterOrEqual": lambda a, b: a >= b, "Equal": lambda a, b: a == b, "NotEqual": lambda a, b: a != b,
        "InSet": lambda a, b: a in b, "NotInSet": lambda a, b: a not in b}


class ColumnCondition:
    def __init__(self, column, op, value): self.column, self.op, self.value = column, op, value
    def bind(self, schema): self.idx = schema.getIndexOfColumn(self.column)
    def condition(self, record): return _OPS[self.op](unwrap(record[self.idx]), self.value)
    def to_dict(self): return {"@class": type(self).__name__, "column": self.column, "op": self.op, "value": list(self.value) if isinstance(self.value, (set, frozenset)) else self.value}


class IntegerColumnCondition(ColumnCondition): pass
class DoubleColumnCondition(ColumnCondition): pass
class StringColumnCondition(ColumnCondition): pass
class CategoricalColumnCondition(ColumnCondition): pass


class NullWritableColumnCondition(ColumnCondition):
    def __init__(self, column): super().__init__(column, "Equal", None)
    def condition(self, record):
        v = unwrap(record[self.idx])
        return v is None or v == ""


class InvalidValueColumnCondition(ColumnCondition):
    def __init__(self, column): super().__init__(column, "Equal", None)
    def bind(self, schema):
        super().bind(schema)
        self.ctype = schema.getType(self.idx)
    def condition(self, record):
        v = unwrap(record[self.idx])
        if self.ctype in (ColumnType.Integer, ColumnType.Long):
            return not isinstance(v, int)
        if self.ctype in (ColumnType.Double, ColumnType.Float):
            return not isinstance(v, (int, float)) or (isinstance(v, float) and (math.isnan(v) or math.isinf(v)))
        return v is None


class BooleanCondition:
    def __init__(self, kind, *conds): self.kind, self.conds = kind, conds
    @staticmethod
    def AND(*c): return BooleanCondition("AND", *c)
    @staticmethod
    def OR(*c): return BooleanCondition("OR", *c)
    @staticmethod
    def NOT(c): return BooleanCondition("NOT", c)
    def bind(self, schema): [c.bind(schema) for c in self.conds]
    def condition(self, r):
        if self.kind == "AND":
            return all(c.condition(r) for c in self.conds)
        if self.kind == "OR":
            return any(c.condition(r) for c in self.conds)
        return not self.conds[0].condition(r)
    def to_dict(self): return {"@class": "BooleanCondition", "kind": self.kind, "conditions": [c.to_dict() for c in self.conds]}


class ConditionFilter:
    """Removes records for which the condition holds."""
    def __init__(self, condition): self.cond = condition


class MathOp:
    Add, Subtract, Multiply, Divide, Modulus, ReverseSubtract, ReverseDivide, ScalarMin, ScalarMax = (
        "Add", "Subtract", "Multiply", "Divide", "Modulus", "ReverseSubtract", "ReverseDivide", "ScalarMin", "ScalarMax")


_MATH = {"Add": lambda a, b: a + b, "Subtract": lambda a, b: a - b, "Multiply": lambda a, b: a * b, "Divide": lambda a, b: a / b,
         "Modulus": lambda a, b: a % b, "ReverseSubtract": lambda a, b: b - a, "ReverseDivide": lambda a, b: b / a,
         "ScalarMin": min, "ScalarMax": max}


class MathFunction:
    ABS, CEIL, EXP, FLOOR, LOG, LOG10, SIGNUM, SIN, COS, TAN, SQRT, TANH = "ABS CEIL EXP FLOOR LOG LOG10 SIGNUM SIN COS TAN SQRT TANH".split()


_FUNCS = {"ABS": abs, "CEIL": math.ceil, "EXP": math.exp, "FLOOR": math.floor, "LOG": math.log, "LOG10": math.log10,
          "SIGNUM": lambda v: (v > 0) - (v < 0), "SIN": math.sin, "COS": math.cos, "TAN": math.tan, "SQRT": math.sqrt, "TANH": math.tanh}


class ReduceOp:
    Min, Max, Range, Sum, Mean, Stdev, Count, CountUnique, TakeFirst, TakeLast, Prod = (
        "Min", "Max", "Range", "Sum", "Mean", "Stdev", "Count", "CountUnique", "TakeFirst", "TakeLast", "Prod")


def _reduce(op, vals):
    if op == "Min": return min(vals)
    if op == "Max": return max(vals)
    if op == "Range": return max(vals) - min(vals)
    if op == "Sum": return sum(vals)
    if op == "Mean": return sum(vals) / len(vals)
    if op == "Stdev":
        m = sum(vals) / len(vals)
        return math.sqrt(sum((v - m) ** 2 for v in vals) / max(len(vals) - 1, 1))
    if op == "Count": return len(vals)
    if op == "CountUnique": return len(set(vals))
    if op == "TakeFirst": return vals[0]
    if op == "TakeLast": return vals[-1]
    if op == "Prod": return math.prod(vals)
    raise ValueError(op)


class Reducer:
    def __init__(self, keyColumns, defaultOp, ops): self.keys, self.defaultOp, self.ops = list(keyColumns), defaultOp, dict(ops)

    class Builder:
        def __init__(self, defaultOp): self.defaultOp, self.keys, self.ops = defaultOp, [], {}
        def keyColumns(self, *k): self.keys = list(k); return self
        def _set(self, op, cols):
            for c in cols:
                self.ops[c] = op
            return self
        def minColumns(self, *c): return self._set("Min", c)
        def maxColumns(self, *c): return self._set("Max", c)
        def sumColumns(self, *c): return self._set("Sum", c)
        def meanColumns(self, *c): return self._set("Mean", c)
        def stdevColumns(self, *c): return self._set("Stdev", c)
        def countColumns(self, *c): return self._set("Count", c)
        def countUniqueColumns(self, *c): return self._set("CountUnique", c)
        def takeFirstColumns(self, *c): return self._set("TakeFirst", c)
        def takeLastColumns(self, *c): return self._set("TakeLast", c)
        def build(self): return Reducer(self.keys, self.defaultOp, self.ops)


_TIME_UNIT_MS = {"MILLISECONDS": 1, "SECONDS": 1000, "MINUTES": 60_000, "HOURS": 3_600_000, "DAYS": 86_400_000}


def _nd_math():
    import numpy as np
    m = {"Add": lambda a, b: a + b, "Subtract": lambda a, b: a - b, "Multiply": lambda a, b: a * b, "Divide": lambda a, b: a / b,
         "Modulus": lambda a, b: np.fmod(a, b), "ReverseSubtract": lambda a, b: b - a, "ReverseDivide": lambda a, b: b / a,
         "ScalarMin": np.minimum, "ScalarMax": np.maximum}
    f = {"ABS": np.abs, "CEIL": np.ceil, "EXP": np.exp, "FLOOR": np.floor, "LOG": np.log, "LOG10": np.log10, "SIGNUM": np.sign, "SIN": np.sin,
         "COS": np.cos, "TAN": np.tan, "SQRT": np.sqrt, "TANH": np.tanh}
    return m, f


_MATH_ND, _FUNCS_ND = _nd_math()


class Distance:
    COSINE, EUCLIDEAN, MANHATTAN = "COSINE", "EUCLIDEAN", "MANHATTAN"


class SplitMaxLengthSequence:
    """``sequence/split/SplitMaxLengthSequence.java``: pieces of at most ``maxSequenceLength`` steps (of equal length when asked)."""
    def __init__(self, maxSequenceLength, equalSplits=False): self.maxSequenceLength, self.equalSplits = int(maxSequenceLength), bool(equalSplits)
    def bind(self, schema): pass
    def split(self, seq):
        n = self.maxSequenceLength
        if len(seq) <= n:
            return [list(seq)]
        size = math.ceil(len(seq) / math.ceil(len(seq) / n)) if self.equalSplits else n
        return [list(seq[k:k + size]) for k in range(0, len(seq), size)]
    def to_dict(self): return {"@class": "SplitMaxLengthSequence", "maxSequenceLength": self.maxSequenceLength, "equalSplits": self.equalSplits}


class SequenceSplitTimeSeparation:
    """``sequence/split/SequenceSplitTimeSeparation.java``: a new sequence starts where two consecutive time stamps are more than the gap apart."""
    def __init__(self, timeColumn, timeQuantity, timeUnit="MILLISECONDS"):
        self.timeColumn, self.timeQuantity, self.timeUnit = timeColumn, int(timeQuantity), str(timeUnit).upper()
    def bind(self, schema): self.idx = schema.getIndexOfColumn(self.timeColumn)
    def split(self, seq):
        gap, out, cur = self.timeQuantity * _TIME_UNIT_MS[self.timeUnit], [], []
        for row in seq:
            if cur and unwrap(row[self.idx]) - unwrap(cur[-1][self.idx]) > gap:
                out.append(cur)
                cur = []
            cur.append(list(row))
        return out + ([cur] if cur else [])
    def to_dict(self): return {"@class": "SequenceSplitTimeSeparation", "timeColumn": self.timeColumn, "timeQuantity": self.timeQuantity, "timeUnit": self.timeUnit}


class TimeWindowFunction:
    """``sequence/window/TimeWindowFunction.java``: consecutive windows of ``windowSize`` starting at ``offset`` past the epoch; a step falls in the
    window that holds its time stamp.  Empty windows between the first and the last are left out unless ``excludeEmptyWindows`` is ``False``."""
    def __init__(self, timeColumn, windowSize, windowSizeUnit="MILLISECONDS", offset=0, offsetUnit="MILLISECONDS", excludeEmptyWindows=True):
        self.timeColumn, self.windowSize, self.windowSizeUnit = timeColumn, int(windowSize), str(windowSizeUnit).upper()
        self.offset, self.offsetUnit, self.excludeEmptyWindows = int(offset), str(offsetUnit).upper(), bool(excludeEmptyWindows)
    def bind(self, schema): self.idx = schema.getIndexOfColumn(self.timeColumn)
    def _ms(self): return self.windowSize * _TIME_UNIT_MS[self.windowSizeUnit], self.offset * _TIME_UNIT_MS[self.offsetUnit]
    def applyToSequence(self, seq):
        if not seq:
            return []
        size, off = self._ms()
        buckets = OrderedDict()
        for row in seq:
            buckets.setdefault((unwrap(row[self.idx]) - off) // size, []).append(row)
        if self.excludeEmptyWindows:
            return list(buckets.values())
        lo, hi = min(buckets), max(buckets)
        return [buckets.get(b, []) for b in range(lo, hi + 1)]
    def to_dict(self):
        return {"@class": "TimeWindowFunction", "timeColumn": self.timeColumn, "windowSize": self.windowSize, "windowSizeUnit": self.windowSizeUnit,
                "offset": self.offset, "offsetUnit": self.offsetUnit, "excludeEmptyWindows": self.excludeEmptyWindows}


class OverlappingTimeWindowFunction(TimeWindowFunction):
    """``sequence/window/OverlappingTimeWindowFunction.java``: windows of ``windowSize`` that start every ``windowSeparation``; a step belongs to
    every window that covers its time stamp."""
    def __init__(self, timeColumn, windowSize, windowSizeUnit, windowSeparation, windowSeparationUnit="MILLISECONDS", offset=0, offsetUnit="MILLISECONDS",
                 excludeEmptyWindows=True):
        super().__init__(timeColumn, windowSize, windowSizeUnit, offset, offsetUnit, excludeEmptyWindows)
        self.windowSeparation, self.windowSeparationUnit = int(windowSeparation), str(windowSeparationUnit).upper()
    def applyToSequence(self, seq):
        if not seq:
            return []
        size, off = self._ms()
        sep = self.windowSeparation * _TIME_UNIT_MS[self.windowSeparationUnit]
        times = [unwrap(r[self.idx]) for r in seq]
        first = (min(times) - off - size) // sep + 1                       # first window whose end lies past the first time stamp
        last = (max(times) - off) // sep
        out = []
        for w in range(first, last + 1):
            lo = off + w * sep
            rows = [r for r, t in zip(seq, times) if lo <= t < lo + size]
            if rows or not self.excludeEmptyWindows:
                out.append(rows)
        return out
    def to_dict(self):
        return dict(super().to_dict(), **{"@class": "OverlappingTimeWindowFunction", "windowSeparation": self.windowSeparation,
                                          "windowSeparationUnit": self.windowSeparationUnit})


# ----------------------------------------------------------------------------- transform process
class _Step:
    def __init__(self, kind, **kw): self.kind, self.kw = kind, kw
    def to_dict(self):
        d = {"kind": self.kind}
        for k, v in self.kw.items():
            d[k] = v.to_dict() if hasattr(v, "to_dict") else (sorted(v) if isinstance(v, (set, frozenset)) else v)
        return d


class TransformProcess:
    def __init__(self, initialSchema, steps):
        self.initialSchema, self.steps = initialSchema, steps
        self._compile()

    class Builder:
        def __init__(self, schema): self.schema, self.steps = schema, []
        def _s(self, kind, **kw): self.steps.append(_Step(kind, **kw)); return self
        def removeColumns(self, *c): return self._s("removeColumns", columns=list(c))
        def removeAllColumnsExceptFor(self, *c): return self._s("keepColumns", columns=list(c))
        def renameColumn(self, old, new): return self._s("rename", old=old, new=new)
        def reorderColumns(self, *c): return self._s("reorder", columns=list(c))
        def duplicateColumn(self, col, newName): return self._s("duplicate", column=col, newName=newName)
        def addConstantIntegerColumn(self, name, v): return self._s("addConstant", name=name, type=ColumnType.Integer, value=v)
        def addConstantDoubleColumn(self, name, v): return self._s("addConstant", name=name, type=ColumnType.Double, value=v)
        def categoricalToInteger(self, *c): return self._s("catToInt", columns=list(c))
        def categoricalToOneHot(self, *c): return self._s("catToOneHot", columns=list(c))
        def integerToCategorical(self, col, states): return self._s("intToCat", column=col, states=list(states))
        def integerToOneHot(self, col, lo, hi): return self._s("intToOneHot", column=col, lo=lo, hi=hi)
        def stringToCategorical(self, col, states): return self._s("strToCat", column=col, states=list(states))
        def convertToString(self, col): return self._s("convert", column=col, to=ColumnType.String)
        def convertToDouble(self, col): return self._s("convert", column=col, to=ColumnType.Double)
        def convertToInteger(self, col): return self._s("convert", column=col, to=ColumnType.Integer)
        def integerMathOp(self, col, op, v): return self._s("math", column=col, op=op, value=v, integer=True)
        def longMathOp(self, col, op, v): return self._s("math", column=col, op=op, value=v, integer=True)
        def doubleMathOp(self, col, op, v): return self._s("math", column=col, op=op, value=v, integer=False)
        floatMathOp = doubleMathOp
        def doubleMathFunction(self, col, fn): return self._s("mathFn", column=col, fn=fn)
        floatMathFunction = doubleMathFunction
        def doubleColumnsMathOp(self, newName, op, *cols): return self._s("columnsMath", newName=newName, op=op, columns=list(cols), integer=False)
        def integerColumnsMathOp(self, newName, op, *cols): return self._s("columnsMath", newName=newName, op=op, columns=list(cols), integer=True)
        def normalize(self, col, kind, stats): return self._s("normalize", column=col, mode=kind, stats=dict(stats))
        def stringMapTransform(self, col, mapping): return self._s("strMap", column=col, mapping=dict(mapping))
        def replaceStringTransform(self, col, mapping): return self._s("strReplace", column=col, mapping=dict(mapping))
        def stringRemoveWhitespaceTransform(self, col): return self._s("strReplace", column=col, mapping={r"\s+": ""})
        def appendStringColumnTransform(self, col, s): return self._s("strAppend", column=col, suffix=s)
        def changeCaseStringTransform(self, col, upper=False): return self._s("strCase", column=col, upper=upper)
        def concatenateStringColumns(self, newName, delim, *cols): return self._s("strConcat", newName=newName, delim=delim, columns=list(cols))
        def conditionalReplaceValueTransform(self, col, newValue, cond): return self._s("condReplace", column=col, value=newValue, condition=cond)
        def conditionalCopyValueTransform(self, col, src, cond): return self._s("condCopy", column=col, source=src, condition=cond)
        def filter(self, f): return self._s("filter", condition=f.cond if isinstance(f, ConditionFilter) else f)
        def stringToTimeTransform(self, col, fmt, tz="UTC"): return self._s("strToTime", column=col, format=fmt, tz=tz)
        def reduce(self, reducer): return self._s("reduce", reducer=reducer)
        def convertToSequence(self, keyColumn, sortColumn=None): return self._s("toSequence", key=keyColumn, sort=sortColumn)
        def offsetSequence(self, cols, offset, kind="InPlace"): return self._s("offsetSeq", columns=list(cols), offset=offset, mode=kind)
        def renameColumns(self, oldNames, newNames):
            for o, n in zip(oldNames, newNames):
                self.renameColumn(o, n)
            return self
        def duplicateColumns(self, columnNames, newNames):
            for c, n in zip(columnNames, newNames):
                self.duplicateColumn(c, n)
            return self
        def addConstantColumn(self, name, columnType, v): return self._s("addConstant", name=name, type=columnType, value=unwrap(v))
        def addConstantLongColumn(self, name, v): return self._s("addConstant", name=name, type=ColumnType.Long, value=int(v))
        def floatMathOp(self, col, op, v): return self._s("math", column=col, op=op, value=v, integer=False)
        def floatMathFunction(self, col, fn): return self._s("mathFn", column=col, fn=fn)
        def floatColumnsMathOp(self, newName, op, *cols): return self._s("columnsMath", newName=newName, op=op, columns=list(cols), integer=False)
        def longColumnsMathOp(self, newName, op, *cols): return self._s("columnsMath", newName=newName, op=op, columns=list(cols), integer=True)
        def timeMathOp(self, col, op, timeQuantity, timeUnit="MILLISECONDS"):
            """``TimeMathOpTransform``: Add / Subtract / ScalarMin / ScalarMax on an epoch-millisecond column, the scalar given in ``timeUnit``."""
            if op not in ("Add", "Subtract", "ScalarMin", "ScalarMax"):
                raise ValueError(f"Invalid MathOp for a time column: {op}")
            return self._s("math", column=col, op=op, value=int(timeQuantity) * _TIME_UNIT_MS[str(timeUnit).upper()], integer=True)
        def conditionalReplaceValueTransformWithDefault(self, col, yesVal, noVal, cond):
            return self._s("condReplaceDefault", column=col, yes=unwrap(yesVal), no=unwrap(noVal), condition=cond)
        def firstDigitTransform(self, inputColumn, outputColumn, mode="INCLUDE_OTHER_CATEGORY"):
            return self._s("firstDigit", column=inputColumn, output=outputColumn, mode=mode)
        def ndArrayScalarOpTransform(self, col, op, v): return self._s("ndScalar", column=col, op=op, value=float(v))
        def ndArrayColumnsMathOpTransform(self, newName, op, *cols): return self._s("ndColumnsMath", newName=newName, op=op, columns=list(cols))
        def ndArrayMathFunctionTransform(self, col, fn): return self._s("ndMathFn", column=col, fn=fn)
        def ndArrayDistanceTransform(self, newName, distance, firstCol, secondCol):
            return self._s("ndDistance", newName=newName, distance=str(distance).upper(), first=firstCol, second=secondCol)
        def calculateSortedRank(self, newColumnName, sortOnColumn, comparator=None, ascending=True):
            """``CalculateSortedRank``: appends a Long column with each record's rank (0 = first) after sorting all records on a column."""
            return self._s("sortedRank", newName=newColumnName, column=sortOnColumn, ascending=bool(ascending))
        def trimSequence(self, numStepsToTrim, trimFromStart=True): return self._s("trimSeq", n=int(numStepsToTrim), fromStart=bool(trimFromStart))
        def trimSequenceToLength(self, maxLength): return self._s("trimSeqToLength", length=int(maxLength), pad=None)
        def trimOrPadSequenceToLength(self, length, pad): return self._s("trimSeqToLength", length=int(length), pad=[unwrap(v) for v in pad])
        def splitSequence(self, split): return self._s("splitSeq", split=split)
        def reduceSequenceByWindow(self, reducer, windowFunction): return self._s("windowReduce", reducer=reducer, window=windowFunction)
        def convertFromSequence(self): return self._s("fromSequence")
        def transform(self, fn): return self._s("custom", fn=fn)
        def build(self): return TransformProcess(self.schema, self.steps)

    # -- compile steps against the evolving schema
    def _compile(self):
        sch = Schema(list(self.initialSchema.columns))
        self._fns, self._global = [], []
        for st in self.steps:
            fn, sch = self._make(st, sch)
            self._fns.append((st.kind, fn))
        self.finalSchema = sch

    def getFinalSchema(self): return self.finalSchema
    def getInitialSchema(self): return self.initialSchema
    def getActionList(self): return list(self.steps)

    @staticmethod
    def _make(st, sch):
        k, kw = st.kind, st.kw
        cols = list(sch.columns)
        ix = sch.getIndexOfColumn
        if k == "removeColumns":
            drop = {ix(c) for c in kw["columns"]}
            return (lambda r: [v for i, v in enumerate(r) if i not in drop]), Schema([c for i, c in enumerate(cols) if i not in drop])
        if k == "keepColumns":
            keep = [ix(c) for c in kw["columns"]]
            ks = sorted(keep)
            return (lambda r: [r[i] for i in ks]), Schema([cols[i] for i in ks])
        if k == "rename":
            i = ix(kw["old"])
            cols[i] = ColumnMeta(kw["new"], cols[i].type, **cols[i].extra)
            return (lambda r: r), Schema(cols)
        if k == "reorder":
            first = [ix(c) for c in kw["columns"]]
            order = first + [i for i in range(len(cols)) if i not in first]
            return (lambda r: [r[i] for i in order]), Schema([cols[i] for i in order])
        if k == "duplicate":
            i = ix(kw["column"])
            return (lambda r: r[:i + 1] + [r[i]] + r[i + 1:]), Schema(cols[:i + 1] + [ColumnMeta(kw["newName"], cols[i].type, **cols[i].extra)] + cols[i + 1:])
        if k == "addConstant":
            v = kw["value"]
            return (lambda r: r + [v]), Schema(cols + [ColumnMeta(kw["name"], kw["type"])])
        if k == "catToInt":
            m = {ix(c): {s: j for j, s in enumerate(sch.getMetaData(c).extra["stateNames"])} for c in kw["columns"]}
            for i in m:
                cols[i] = ColumnMeta(cols[i].name, ColumnType.Integer)
            return (lambda r: [m[i][str(unwrap(v))] if i in m else v for i, v in enumerate(r)]), Schema(cols)
        if k == "catToOneHot":
            m = {ix(c): sch.getMetaData(c).extra["stateNames"] for c in kw["columns"]}
            new = []
            for i, c in enumerate(cols):
                new += [ColumnMeta(f"{c.name}[{s}]", ColumnType.Integer) for s in m[i]] if i in m else [c]
            def f(r):
                out = []
                for i, v in enumerate(r):
                    if i in m:
                        s = str(unwrap(v))
                        if s not in m[i]:
                            raise ValueError(f"unknown state {s!r} for categorical column {cols[i].name}")
                        out += [1 if s == t else 0 for t in m[i]]
                    else:
                        out.append(v)
                return out
            return f, Schema(new)
        if k == "intToCat":
            i, states = ix(kw["column"]), kw["states"]
            cols[i] = ColumnMeta(cols[i].name, ColumnType.Categorical, stateNames=states)
            return (lambda r: r[:i] + [states[int(unwrap(r[i]))]] + r[i + 1:]), Schema(cols)
        if k == "intToOneHot":
            i, lo, hi = ix(kw["column"]), kw["lo"], kw["hi"]
            new = cols[:i] + [ColumnMeta(f"{cols[i].name}[{v}]", ColumnType.Integer) for v in range(lo, hi + 1)] + cols[i + 1:]
            return (lambda r: r[:i] + [1 if int(unwrap(r[i])) == v else 0 for v in range(lo, hi + 1)] + r[i + 1:]), Schema(new)
        if k == "strToCat":
            i = ix(kw["column"])
            cols[i] = ColumnMeta(cols[i].name, ColumnType.Categorical, stateNames=kw["states"])
            return (lambda r: r), Schema(cols)
        if k == "convert":
            i, to = ix(kw["column"]), kw["to"]
            conv = {ColumnType.String: str, ColumnType.Double: float, ColumnType.Integer: lambda v: int(float(v))}[to]
            cols[i] = ColumnMeta(cols[i].name, to)
            return (lambda r: r[:i] + [conv(unwrap(r[i]))] + r[i + 1:]), Schema(cols)
        if k == "math":
            i, op, b, integer = ix(kw["column"]), _MATH[kw["op"]], kw["value"], kw["integer"]
            def f(r):
                v = op(unwrap(r[i]), b)
                return r[:i] + [int(v) if integer else float(v)] + r[i + 1:]
            return f, sch
        if k == "mathFn":
            i, fn = ix(kw["column"]), _FUNCS[kw["fn"]]
            return (lambda r: r[:i] + [float(fn(unwrap(r[i])))] + r[i + 1:]), sch
        if k == "columnsMath":
            idx, op, integer = [ix(c) for c in kw["columns"]], _MATH[kw["op"]], kw["integer"]
            def f(r):
                v = unwrap(r[idx[0]])
                for j in idx[1:]:
                    v = op(v, unwrap(r[j]))
                return r + [int(v) if integer else float(v)]
            return f, Schema(cols + [ColumnMeta(kw["newName"], ColumnType.Integer if integer else ColumnType.Double)])
        if k == "normalize":
            i, mode, s = ix(kw["column"]), kw["mode"], kw["stats"]
            if mode in ("Standardize", "standardize"):
                g = lambda v: (v - s["mean"]) / (s["stdev"] or 1.0)
            elif mode in ("MinMax", "minmax"):
                g = lambda v: (v - s["min"]) / ((s["max"] - s["min"]) or 1.0)
            elif mode in ("Log2Mean", "log2mean"):
                g = lambda v: math.log2((v - s["min"]) / (s["mean"] - s["min"]) + 1)
            else:
                raise ValueError(mode)
            return (lambda r: r[:i] + [g(float(unwrap(r[i])))] + r[i + 1:]), sch
        if k == "strMap":
            i, m = ix(kw["column"]), kw["mapping"]
            return (lambda r: r[:i] + [m.get(str(unwrap(r[i])), unwrap(r[i]))] + r[i + 1:]), sch
        if k == "strReplace":
            i, m = ix(kw["column"]), [(re.compile(a), b) for a, b in kw["mapping"].items()]
            def f(r):
                s = str(unwrap(r[i]))
                for rx, b in m:
                    s = rx.sub(b, s)
                return r[:i] + [s] + r[i + 1:]
            return f, sch
        if k == "strAppend":
            i, suf = ix(kw["column"]), kw["suffix"]
            return (lambda r: r[:i] + [str(unwrap(r[i])) + suf] + r[i + 1:]), sch
        if k == "strCase":
            i, up = ix(kw["column"]), kw["upper"]
            return (lambda r: r[:i] + [str(unwrap(r[i])).upper() if up else str(unwrap(r[i])).lower()] + r[i + 1:]), sch
        if k == "strConcat":
            idx, d = [ix(c) for c in kw["columns"]], kw["delim"]
            return (lambda r: r + [d.join(str(unwrap(r[j])) for j in idx)]), Schema(cols + [ColumnMeta(kw["newName"], ColumnType.String)])
        if k == "condReplace":
            i, v, c = ix(kw["column"]), kw["value"], kw["condition"]
            c.bind(sch)
            return (lambda r: r[:i] + [v] + r[i + 1:] if c.condition(r) else r), sch
        if k == "condCopy":
            i, j, c = ix(kw["column"]), ix(kw["source"]), kw["condition"]
            c.bind(sch)
            return (lambda r: r[:i] + [r[j]] + r[i + 1:] if c.condition(r) else r), sch
        if k == "filter":
            c = kw["condition"]
            c.bind(sch)
            return (lambda r: None if c.condition(r) else r), sch
        if k == "strToTime":
            import calendar
            import time as _time
            i, fmt = ix(kw["column"]), kw["format"]
            pyfmt = fmt.replace("yyyy", "%Y").replace("MM", "%m").replace("dd", "%d").replace("HH", "%H").replace("mm", "%M").replace("ss", "%S")
            cols[i] = ColumnMeta(cols[i].name, ColumnType.Time, timeZone=kw["tz"])
            return (lambda r: r[:i] + [calendar.timegm(_time.strptime(str(unwrap(r[i])), pyfmt)) * 1000] + r[i + 1:]), Schema(cols)
        if k == "custom":
            return kw["fn"], sch
        if k == "reduce":
            red = kw["reducer"]
            keys = [ix(c) for c in red.keys]
            new = []
            for i, c in enumerate(cols):
                if i in keys:
                    new.append(c)
                else:
                    op = red.ops.get(c.name, red.defaultOp)
                    t = ColumnType.Long if op in ("Count", "CountUnique") else (ColumnType.Double if op in ("Mean", "Stdev") else c.type)
                    new.append(ColumnMeta(f"{op.lower()}({c.name})", t))
            return ("GLOBAL", red, keys, [c.name for c in cols]), Schema(new)
        if k in ("toSequence", "offsetSeq"):
            return ("GLOBAL", k, kw, [c.name for c in cols]), sch
        if k == "condReplaceDefault":
            i, yes, no, c = ix(kw["column"]), kw["yes"], kw["no"], kw["condition"]
            c.bind(sch)
            return (lambda r: r[:i] + [yes if c.condition(r) else no] + r[i + 1:]), sch
        if k == "firstDigit":
            i, outn, mode = ix(kw["column"]), kw["output"], kw["mode"]
            states = [str(d) for d in range(10)] + (["Other"] if mode == "INCLUDE_OTHER_CATEGORY" else [])
            def digit(v):
                t = str(unwrap(v))
                t = t[1:] if t.startswith("-") and len(t) > 1 else t
                if t and t[0].isdigit():
                    return t[0]
                if mode == "INCLUDE_OTHER_CATEGORY":
                    return "Other"
                raise ValueError(f"FirstDigitTransform in mode EXCEPTION_ON_INVALID met the non-numerical entry {unwrap(v)!r}")
            meta = ColumnMeta(outn, ColumnType.Categorical, stateNames=states)
            if outn == kw["column"]:
                cols[i] = meta
                return (lambda r: r[:i] + [digit(r[i])] + r[i + 1:]), Schema(cols)
            return (lambda r: r[:i + 1] + [digit(r[i])] + r[i + 1:]), Schema(cols[:i + 1] + [meta] + cols[i + 1:])
        if k in ("ndScalar", "ndMathFn", "ndColumnsMath", "ndDistance"):
            import numpy as np
            A = lambda v: np.asarray(unwrap(v), dtype=np.float64)
            if k == "ndScalar":
                i, op, b = ix(kw["column"]), _MATH_ND[kw["op"]], kw["value"]
                return (lambda r: r[:i] + [op(A(r[i]), b)] + r[i + 1:]), sch
            if k == "ndMathFn":
                i, fn = ix(kw["column"]), _FUNCS_ND[kw["fn"]]
                return (lambda r: r[:i] + [fn(A(r[i]))] + r[i + 1:]), sch
            if k == "ndColumnsMath":
                if kw["op"] not in ("Add", "Subtract", "Multiply", "Divide"):
                    raise ValueError(f"Invalid MathOp for NDArray columns: {kw['op']}")
                idx, op = [ix(c) for c in kw["columns"]], _MATH_ND[kw["op"]]
                def f(r):
                    v = A(r[idx[0]])
                    for j in idx[1:]:
                        v = op(v, A(r[j]))
                    return r + [v]
                return f, Schema(cols + [ColumnMeta(kw["newName"], ColumnType.NDArray, **cols[idx[0]].extra)])
            a, b, d = ix(kw["first"]), ix(kw["second"]), kw["distance"]
            def dist(x, y):
                if d == "COSINE":
                    return float(1.0 - (x * y).sum() / (np.linalg.norm(x) * np.linalg.norm(y)))
                if d == "EUCLIDEAN":
                    return float(np.linalg.norm(x - y))
                if d == "MANHATTAN":
                    return float(np.abs(x - y).sum())
                raise ValueError(f"unknown distance {d}")
            return (lambda r: r + [dist(A(r[a]).ravel(), A(r[b]).ravel())]), Schema(cols + [ColumnMeta(kw["newName"], ColumnType.Double)])
        if k == "sortedRank":
            i, asc = ix(kw["column"]), kw["ascending"]
            def rank(rows):
                order = sorted(range(len(rows)), key=lambda j: unwrap(rows[j][i]), reverse=not asc)
                pos = {j: n for n, j in enumerate(order)}
                return [list(r) + [pos[j]] for j, r in enumerate(rows)]
            return ("GLOBAL", "rowsFn", rank, None), Schema(cols + [ColumnMeta(kw["newName"], ColumnType.Long)])
        if k == "trimSeq":
            n, start = kw["n"], kw["fromStart"]
            return ("GLOBAL", "rowsFn", lambda seqs: [s[n:] if start else s[:max(len(s) - n, 0)] for s in seqs], None), sch
        if k == "trimSeqToLength":
            n, pad = kw["length"], kw["pad"]
            if pad is not None and len(pad) != len(cols):
                raise ValueError(f"the padding record has {len(pad)} values for {len(cols)} columns")
            return ("GLOBAL", "rowsFn", lambda seqs: [list(s[:n]) + ([list(pad) for _ in range(n - len(s))] if pad is not None else []) for s in seqs], None), sch
        if k == "splitSeq":
            sp = kw["split"]
            sp.bind(sch)
            return ("GLOBAL", "rowsFn", lambda seqs: [piece for s in seqs for piece in sp.split(s)], None), sch
        if k == "fromSequence":
            return ("GLOBAL", "rowsFn", lambda seqs: [list(r) for s in seqs for r in s], None), sch
        if k == "windowReduce":
            red, win = kw["reducer"], kw["window"]
            win.bind(sch)
            names = [c.name for c in cols]
            new = []
            for c in cols:
                op = red.ops.get(c.name, red.defaultOp)
                t = ColumnType.Long if op in ("Count", "CountUnique") else (ColumnType.Double if op in ("Mean", "Stdev") else c.type)
                new.append(ColumnMeta(f"{op.lower()}({c.name})", t))
            def f(seqs):
                out = []
                for s in seqs:
                    steps = []
                    for w in win.applyToSequence(s):
                        ops = [red.ops.get(n, red.defaultOp) for n in names]
                        if w:
                            steps.append([_reduce(op, [unwrap(r[i]) for r in w]) for i, op in enumerate(ops)])
                        else:                                   # an empty window kept on request: counts are 0, everything else is missing
                            steps.append([0 if op in ("Count", "CountUnique") else None for op in ops])
                    out.append(steps)
                return out
            return ("GLOBAL", "rowsFn", f, None), Schema(new)
        raise ValueError(f"unknown transform step {k}")

    # -- execution
    def execute(self, record):
        """Applies the per-record steps to one record (steps that need all records raise); returns None when filtered out."""
        r = list(record)
        for kind, fn in self._fns:
            if isinstance(fn, tuple):
                raise ValueError(f"step '{kind}' needs the whole dataset: use LocalTransformExecutor.execute")
            r = fn(r)
            if r is None:
                return None
        return r

    def executeAll(self, records):
        rows = [list(r) for r in records]
        for kind, fn in self._fns:
            if isinstance(fn, tuple) and fn[1].__class__ is Reducer:
                _, red, keys, names = fn
                groups = OrderedDict()
                for r in rows:
                    groups.setdefault(tuple(unwrap(r[i]) for i in keys), []).append(r)
                out = []
                for key, grp in groups.items():
                    row = []
                    for i, n in enumerate(names):
                        if i in keys:
                            row.append(grp[0][i])
                        else:
                            row.append(_reduce(red.ops.get(n, red.defaultOp), [unwrap(g[i]) for g in grp]))
                    out.append(row)
                rows = out
            elif isinstance(fn, tuple) and fn[1] == "toSequence":
                kw, names = fn[2], fn[3]
                ki = names.index(kw["key"])
                groups = OrderedDict()
                for r in rows:
                    groups.setdefault(unwrap(r[ki]), []).append(r)
                if kw["sort"] is not None:
                    si = names.index(kw["sort"])
                    for g in groups.values():
                        g.sort(key=lambda r: unwrap(r[si]))
                rows = list(groups.values())
            elif isinstance(fn, tuple) and fn[1] == "rowsFn":
                rows = fn[2](rows)
            elif isinstance(fn, tuple) and fn[1] == "offsetSeq":
                kw, names = fn[2], fn[3]
                idx, off = [names.index(c) for c in kw["columns"]], kw["offset"]
                new = []
                for seq in rows:
                    T = len(seq)
                    out = []
                    for t in range(T):
                        s = t - off
                        if 0 <= s < T:
                            out.append([seq[s][i] if i in idx else v for i, v in enumerate(seq[t])])
                    new.append(out)
                rows = new
            else:
                if rows and rows[0] and isinstance(rows[0][0], list):            # sequences: apply per step
                    rows = [[x for x in (fn(list(s)) for s in seq) if x is not None] for seq in rows]
                else:
                    rows = [x for x in (fn(r) for r in rows) if x is not None]
        return rows

    def toJson(self):
        steps = []
        for s in self.steps:
            if s.kind == "custom":
                raise ValueError("custom function steps cannot be serialised")
            d = s.to_dict()
            if s.kind in ("reduce", "windowReduce"):
                r = s.kw["reducer"]
                d["reducer"] = {"keys": r.keys, "defaultOp": r.defaultOp, "ops": r.ops}
            steps.append(d)
        return json.dumps({"initialSchema": json.loads(self.initialSchema.toJson()), "actionList": steps})

    @staticmethod
    def fromJson(s):
        d = json.loads(s)
        sch = Schema.fromJson(json.dumps(d["initialSchema"]))
        def cond(c):
            if c["@class"] == "BooleanCondition":
                return BooleanCondition(c["kind"], *[cond(x) for x in c["conditions"]])
            cls = globals()[c["@class"]]
            if cls in (NullWritableColumnCondition, InvalidValueColumnCondition):
                return cls(c["column"])
            v = c["value"]
            return cls(c["column"], c["op"], set(v) if c["op"] in ("InSet", "NotInSet") else v)
        steps = []
        for st in d["actionList"]:
            kind = st.pop("kind")
            if "condition" in st:
                st["condition"] = cond(st["condition"])
            if kind in ("reduce", "windowReduce"):
                r = st["reducer"]
                st["reducer"] = Reducer(r["keys"], r["defaultOp"], r["ops"])
            for key in ("split", "window"):
                if key in st:
                    spec = dict(st[key])
                    st[key] = globals()[spec.pop("@class")](**spec)
            steps.append(_Step(kind, **st))
        return TransformProcess(sch, steps)


class LocalTransformExecutor:
    @staticmethod
    def execute(records, tp): return tp.executeAll(records)
    executeToSequence = execute


class DataAnalysis:
    """Per-column summary statistics (``AnalyzeLocal.analyze``)."""

    def __init__(self, schema, stats): self.schema, self.stats = schema, stats
    def getColumnAnalysis(self, name): return self.stats[name]
    def __repr__(self): return "\n".join(f"{k}: {v}" for k, v in self.stats.items())


class AnalyzeLocal:
    @staticmethod
    def analyze(schema, records):
        rows = [[unwrap(v) for v in r] for r in records]
        stats = {}
        for i, c in enumerate(schema.columns):
            col = [r[i] for r in rows]
            if c.type in (ColumnType.Integer, ColumnType.Long, ColumnType.Double, ColumnType.Float, ColumnType.Time):
                nums = [float(v) for v in col if isinstance(v, (int, float))]
                m = sum(nums) / max(len(nums), 1)
                stats[c.name] = {"count": len(col), "countInvalid": len(col) - len(nums), "min": min(nums, default=None), "max": max(nums, default=None), "mean": m,
                                 "stdev": math.sqrt(sum((v - m) ** 2 for v in nums) / max(len(nums) - 1, 1)), "countZero": sum(v == 0 for v in nums)}
            else:
                cnt = {}
                for v in col:
                    cnt[str(v)] = cnt.get(str(v), 0) + 1
                stats[c.name] = {"count": len(col), "countUnique": len(cnt), "mapOfCounts": cnt}
        return DataAnalysis(schema, stats)
