"""``TransformProcess.Builder`` steps (``datavec-api/.../transform/TransformProcess.java``) beyond the basic column operations: each
step is checked against the definition of its transform class on a small table."""
import numpy as np
import pytest

from deeplearning4j_b200.datavec import (ColumnCondition, ColumnType, ConditionOp, Distance, LocalTransformExecutor, MathFunction, MathOp,
                                         OverlappingTimeWindowFunction, ReduceOp, Reducer, Schema, SequenceSplitTimeSeparation,
                                         SplitMaxLengthSequence, TimeWindowFunction, TransformProcess)


def test_column_steps():
    sch = Schema.Builder().addColumnString("id").addColumnDouble("x").addColumnLong("n").addColumnTime("t").build()
    tp = (TransformProcess.Builder(sch)
          .renameColumns(["x", "n"], ["value", "count"])
          .duplicateColumns(["value", "count"], ["value2", "count2"])
          .addConstantColumn("who", ColumnType.String, "me").addConstantLongColumn("big", 1 << 40)
          .floatMathOp("value", MathOp.Multiply, 2.0).floatMathFunction("value2", MathFunction.ABS)
          .longColumnsMathOp("total", MathOp.Add, "count", "count2").floatColumnsMathOp("prod", MathOp.Multiply, "value", "value2")
          .timeMathOp("t", MathOp.Add, 2, "HOURS")
          .conditionalReplaceValueTransformWithDefault("who", "neg", "pos", ColumnCondition("value", ConditionOp.LessThan, 0.0))
          .firstDigitTransform("value2", "digit")
          .build())
    assert tp.getFinalSchema().getColumnNames() == ["id", "value", "value2", "digit", "count", "count2", "t", "who", "big", "total", "prod"]
    assert tp.getFinalSchema().getMetaData("digit").extra["stateNames"][-1] == "Other"
    row = tp.execute(["a", -1.5, 3, 1000])
    assert row == ["a", -3.0, 1.5, "1", 3, 3, 1000 + 2 * 3_600_000, "neg", 1 << 40, 6, -4.5]
    assert tp.execute(["b", 0.25, 1, 0])[7] == "pos"
    again = TransformProcess.fromJson(tp.toJson())
    assert again.execute(["a", -1.5, 3, 1000]) == row
    with pytest.raises(ValueError, match="time column"):
        TransformProcess.Builder(sch).timeMathOp("t", MathOp.Multiply, 2)
    strict = TransformProcess.Builder(Schema.Builder().addColumnString("s").build()).firstDigitTransform("s", "s", "EXCEPTION_ON_INVALID").build()
    assert strict.execute(["-42"]) == ["4"]
    with pytest.raises(ValueError, match="non-numerical"):
        strict.execute(["x1"])


def test_ndarray_steps():
    sch = Schema.Builder().addColumnNDArray("a", [3]).addColumnNDArray("b", [3]).build()
    tp = (TransformProcess.Builder(sch)
          .ndArrayScalarOpTransform("a", MathOp.Multiply, 2.0)
          .ndArrayMathFunctionTransform("b", MathFunction.ABS)
          .ndArrayColumnsMathOpTransform("sum", MathOp.Add, "a", "b")
          .ndArrayDistanceTransform("d2", Distance.EUCLIDEAN, "a", "b")
          .ndArrayDistanceTransform("d1", Distance.MANHATTAN, "a", "b")
          .ndArrayDistanceTransform("dc", Distance.COSINE, "a", "b")
          .build())
    a, b = np.array([1.0, 2.0, 3.0]), np.array([-1.0, 0.5, 2.0])
    r = tp.execute([a, b])
    assert np.allclose(r[0], 2 * a) and np.allclose(r[1], np.abs(b)) and np.allclose(r[2], 2 * a + np.abs(b))
    x, y = 2 * a, np.abs(b)
    assert r[3] == pytest.approx(np.linalg.norm(x - y)) and r[4] == pytest.approx(np.abs(x - y).sum())
    assert r[5] == pytest.approx(1 - x @ y / np.linalg.norm(x) / np.linalg.norm(y))
    assert tp.getFinalSchema().getColumnTypes()[2:] == [ColumnType.NDArray, ColumnType.Double, ColumnType.Double, ColumnType.Double]
    assert TransformProcess.fromJson(tp.toJson()).execute([a, b])[3] == pytest.approx(r[3])


def test_sorted_rank_and_sequence_steps():
    sch = Schema.Builder().addColumnString("k").addColumnTime("t").addColumnDouble("v").build()
    rows = [["a", 0, 5.0], ["a", 1000, 1.0], ["a", 2500, 3.0], ["b", 100, 2.0], ["a", 9000, 4.0], ["b", 200, 8.0]]
    ranked = LocalTransformExecutor.execute(rows, TransformProcess.Builder(sch).calculateSortedRank("rank", "v").build())
    assert [r[-1] for r in ranked] == [4, 0, 2, 1, 3, 5]
    ranked = LocalTransformExecutor.execute(rows, TransformProcess.Builder(sch).calculateSortedRank("rank", "v", ascending=False).build())
    assert [r[-1] for r in ranked] == [1, 5, 3, 4, 2, 0]

    base = TransformProcess.Builder(sch).convertToSequence("k", "t")
    seqs = LocalTransformExecutor.execute(rows, base.build())
    assert [len(s) for s in seqs] == [4, 2]

    def run(extend):
        b = TransformProcess.Builder(sch).convertToSequence("k", "t")
        tp = extend(b).build()
        out = LocalTransformExecutor.execute(rows, tp)
        assert LocalTransformExecutor.execute(rows, TransformProcess.fromJson(tp.toJson())) == out     # the steps survive the JSON form
        return out, tp

    out, _ = run(lambda b: b.trimSequence(1, True))
    assert [[r[1] for r in s] for s in out] == [[1000, 2500, 9000], [200]]
    out, _ = run(lambda b: b.trimSequence(3, False))
    assert [[r[1] for r in s] for s in out] == [[0], []]
    out, _ = run(lambda b: b.trimSequenceToLength(3))
    assert [len(s) for s in out] == [3, 2]
    out, _ = run(lambda b: b.trimOrPadSequenceToLength(3, ["pad", -1, 0.0]))
    assert [len(s) for s in out] == [3, 3] and out[1][2] == ["pad", -1, 0.0]
    with pytest.raises(ValueError, match="padding record"):
        run(lambda b: b.trimOrPadSequenceToLength(3, ["pad"]))
    out, _ = run(lambda b: b.splitSequence(SplitMaxLengthSequence(3)))
    assert [len(s) for s in out] == [3, 1, 2]
    out, _ = run(lambda b: b.splitSequence(SplitMaxLengthSequence(3, True)))
    assert [len(s) for s in out] == [2, 2, 2]
    out, _ = run(lambda b: b.splitSequence(SequenceSplitTimeSeparation("t", 2, "SECONDS")))
    assert [[r[1] for r in s] for s in out] == [[0, 1000, 2500], [9000], [100, 200]]
    out, _ = run(lambda b: b.splitSequence(SplitMaxLengthSequence(3)).convertFromSequence())
    assert len(out) == 6 and out[0] == ["a", 0, 5.0]

    red = Reducer.Builder(ReduceOp.TakeFirst).sumColumns("v").build()
    out, tp = run(lambda b: b.reduceSequenceByWindow(red, TimeWindowFunction("t", 2, "SECONDS")))
    assert tp.getFinalSchema().getColumnNames() == ["takefirst(k)", "takefirst(t)", "sum(v)"]
    assert out == [[["a", 0, 6.0], ["a", 2500, 3.0], ["a", 9000, 4.0]], [["b", 100, 10.0]]]
    out, _ = run(lambda b: b.reduceSequenceByWindow(red, TimeWindowFunction("t", 2, "SECONDS", excludeEmptyWindows=False)))
    assert len(out[0]) == 5 and out[0][2] == [None, None, None] and out[0][4] == ["a", 9000, 4.0]
    # overlapping: 2 s windows every second; the step at 1000 ms sits in the windows starting at 0 and at 1000
    out, _ = run(lambda b: b.reduceSequenceByWindow(red, OverlappingTimeWindowFunction("t", 2, "SECONDS", 1, "SECONDS")))
    assert [r[2] for r in out[0]] == [5.0, 6.0, 4.0, 3.0, 4.0, 4.0]
