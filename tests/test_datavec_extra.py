"""Joins, sequence operations, quality analysis, Arrow / JDBC / Excel readers and the image loader + transforms."""
import math
import sqlite3

import numpy as np
import pytest
import torch

from deeplearning4j_b200.datavec import (AnalyzeLocal, ArrowConverter, ArrowRecordReader, ArrowRecordWriter, BoxImageTransform,
                                         ColorConversionTransform, ColumnType, CropImageTransform, EqualizeHistTransform,
                                         ExcelRecordReader, ExcelRecordWriter, FileSplit, FlipImageTransform, JDBCRecordReader, Join,
                                         JoinType, LocalTransformExecutor, NativeImageLoader, PipelineImageTransform,
                                         RandomCropTransform, Reducer, ResizeImageTransform, RotateImageTransform, Schema,
                                         convertFromSequence, reduceSequence, sequenceDifference, sequenceMovingWindowReduce,
                                         splitSequenceMaxLength, splitSequenceTimeSeparation, trimSequence, trimSequenceToLength)


def _schemas():
    left = Schema.Builder().addColumnInteger("id").addColumnString("name").build()
    right = Schema.Builder().addColumnInteger("id").addColumnDouble("amount").build()
    return left, right


def test_joins_of_all_four_kinds():
    left, right = _schemas()
    L = [[1, "ann"], [2, "bob"], [3, "cyd"]]
    R = [[1, 10.0], [1, 11.0], [3, 30.0], [4, 40.0]]
    j = Join.Builder(JoinType.Inner).setSchemas(left, right).setJoinColumns("id").build()
    assert j.getOutputSchema().getColumnNames() == ["id", "name", "amount"]
    assert LocalTransformExecutor.executeJoin(j, L, R) == [[1, "ann", 10.0], [1, "ann", 11.0], [3, "cyd", 30.0]]
    lo = Join.Builder(JoinType.LeftOuter).setSchemas(left, right).setJoinColumns("id").build().execute(L, R)
    assert [2, "bob", None] in lo and len(lo) == 4
    ro = Join.Builder(JoinType.RightOuter).setSchemas(left, right).setJoinColumns("id").build().execute(L, R)
    assert [4, None, 40.0] in ro and [2, "bob", None] not in ro and len(ro) == 4
    fo = Join.Builder(JoinType.FullOuter).setSchemas(left, right).setJoinColumns("id").build().execute(L, R)
    assert len(fo) == 5 and [4, None, 40.0] in fo and [2, "bob", None] in fo
    other = Schema.Builder().addColumnInteger("key").addColumnDouble("amount").build()
    j2 = Join.Builder(JoinType.Inner).setSchemas(left, other).setJoinColumnsLeft("id").setJoinColumnsRight("key").build()
    assert j2.execute(L, R)[0] == [1, "ann", 10.0]
    with pytest.raises(ValueError):
        Join.Builder(JoinType.Inner).setSchemas(left, left).setJoinColumns("id").build().getOutputSchema()


def test_sequence_operations():
    sch = Schema.Builder().addColumnLong("t").addColumnDouble("x").build()
    seqs = [[[0, 1.0], [1, 3.0], [2, 6.0], [10, 10.0], [11, 15.0]], [[0, 2.0], [1, 2.5]]]
    assert [len(s) for s in trimSequence(seqs, 1)] == [4, 1] and trimSequence(seqs, 1, fromFirst=False)[0][-1] == [10, 10.0]
    assert [len(s) for s in trimSequenceToLength(seqs, 3, pad=True)] == [3, 3]
    d = sequenceDifference(sch, seqs, "x")
    assert [r[1] for r in d[0]] == [0, 2.0, 3.0, 4.0, 5.0]
    w, sch2 = sequenceMovingWindowReduce(sch, seqs, "x", 2, "Mean")
    assert sch2.getColumnNames()[-1] == "mean(2,x)" and [r[2] for r in w[0]] == [1.0, 2.0, 4.5, 8.0, 12.5]
    red = Reducer.Builder("Max").sumColumns("x").build()
    assert reduceSequence(sch, seqs, red) == [[11, 35.0], [1, 4.5]]
    assert len(convertFromSequence(seqs)) == 7
    assert [len(s) for s in splitSequenceMaxLength(seqs, 2)] == [2, 2, 1, 2]
    assert [len(s) for s in splitSequenceMaxLength(seqs, 3, equalSplits=True)] == [3, 2, 2]
    assert [len(s) for s in splitSequenceTimeSeparation(sch, seqs, "t", 5)] == [3, 2, 2]


def test_quality_analysis_counts():
    sch = (Schema.Builder().addColumnInteger("i").addColumnDouble("d").addColumnString("s")
           .addColumnCategorical("c", ["a", "b"]).build())
    recs = [[1, 1.5, "x", "a"], ["2", float("nan"), "", "b"], [2.5, float("inf"), "x", "z"], [None, "oops", "y", "a"]]
    q = AnalyzeLocal.analyzeQuality(sch, recs)
    qi, qd, qs, qc = (q.getColumnQuality(n) for n in "idsc")
    assert (qi.countValid, qi.countNonInteger, qi.countMissing, qi.countTotal) == (2, 1, 1, 4)
    assert (qd.countValid, qd.countNaN, qd.countInfinite, qd.countNonNumeric) == (1, 1, 1, 1)
    assert (qs.countEmptyString, qs.countUnique, qs.countValid) == (1, 3, 4)
    assert (qc.countValid, qc.countInvalid) == (3, 1)


def test_arrow_round_trip_and_reader(tmp_path):
    sch = Schema.Builder().addColumnInteger("i").addColumnDouble("d").addColumnString("s").addColumnLong("l").build()
    recs = [[1, 0.5, "a", 10 ** 12], [2, 1.5, "b", 7], [3, -2.0, None, 0]]
    p = str(tmp_path / "r.arrow")
    w = ArrowRecordWriter(sch, p)
    w.writeBatch(recs)
    w.close()
    sch2, back = ArrowConverter.readFromFile(p)
    assert back == recs and sch2.getColumnNames() == ["i", "d", "s", "l"]
    assert [c.type for c in sch2.columns] == [ColumnType.Integer, ColumnType.Double, ColumnType.String, ColumnType.Long]
    rr = ArrowRecordReader()
    rr.initialize(FileSplit(p))
    got = []
    while rr.hasNext():
        got.append(rr.next())
    assert got == recs
    t = ArrowConverter.toTensor(ArrowConverter.toArrowTable(sch, recs).select(["i", "d"]))
    assert t.tolist() == [[1, 0.5], [2, 1.5], [3, -2.0]]


def test_jdbc_reader_over_sqlite():
    con = sqlite3.connect(":memory:")
    con.execute("create table coffee (id integer primary key, name text, price real)")
    con.executemany("insert into coffee values (?, ?, ?)", [(1, "espresso", 2.5), (2, "latte", 3.5), (3, "mocha", 4.0)])
    rr = JDBCRecordReader("select id, name, price from coffee order by id", connection=con,
                          metaDataQuery="select id, name, price from coffee where id = ?", metaDataIndices=[0])
    rr.initialize()
    assert rr.getLabels() == ["id", "name", "price"]
    rows = []
    while rr.hasNext():
        rows.append(rr.next())
    assert rows == [[1, "espresso", 2.5], [2, "latte", 3.5], [3, "mocha", 4.0]]
    rr.reset()
    rec, meta = rr.nextRecordWithMeta()
    assert meta == [1] and rr.loadFromMetaData([3]) == [3, "mocha", 4.0]
    rr.close()


def test_excel_writer_and_reader(tmp_path):
    p = str(tmp_path / "book.xlsx")
    w = ExcelRecordWriter(p)
    w.writeBatch([["id", "name", "score", "ok"], [1, "a & b", 2.5, True], [2, "<c>", -1.0, False], [3, None, 1e-3, True]])
    w.close()
    rr = ExcelRecordReader(skipNumLines=1)
    rr.initialize(FileSplit(p))
    rows = []
    while rr.hasNext():
        rows.append(rr.next())
    assert rows == [[1, "a & b", 2.5, True], [2, "<c>", -1.0, False], [3, None, 0.001, True]]


def test_image_loader_and_transforms(tmp_path):
    from PIL import Image
    rgb = np.zeros((20, 30, 3), dtype=np.uint8)
    rgb[:, :15, 0] = 255
    rgb[:, 15:, 2] = 200
    p = str(tmp_path / "img.png")
    Image.fromarray(rgb).save(p)
    m = NativeImageLoader(10, 12, 3).asMatrix(p)
    assert tuple(m.shape) == (1, 3, 10, 12) and float(m[0, 0, :, 0].mean()) == 255.0 and float(m[0, 2, :, -1].mean()) == 200.0
    g = NativeImageLoader(20, 30, 1).asMatrix(p)
    assert tuple(g.shape) == (1, 1, 20, 30) and abs(float(g[0, 0, 0, 0]) - 0.299 * 255) < 1e-3
    assert tuple(NativeImageLoader(4, 4, 3).asRowVector(p).shape) == (1, 48)
    sq = NativeImageLoader(10, 10, 3, centerCropIfNeeded=True).asMatrix(p)
    assert tuple(sq.shape) == (1, 3, 10, 10)
    out = str(tmp_path / "o.png")
    NativeImageLoader.asFile(m, out)
    assert tuple(NativeImageLoader().asMatrix(out).shape) == (1, 3, 10, 12)
    t = torch.from_numpy(rgb).permute(2, 0, 1).float()
    assert torch.equal(FlipImageTransform(1).transform(t), t.flip(2)) and torch.equal(FlipImageTransform(0).transform(t), t.flip(1))
    assert tuple(CropImageTransform(2, 3).transform(t).shape) == (3, 16, 24)
    assert tuple(RandomCropTransform(8, 9, seed=1).transform(t).shape) == (3, 8, 9)
    assert tuple(ResizeImageTransform(7, 5).transform(t).shape) == (3, 5, 7)
    r0 = RotateImageTransform(0.0, fixed=True).transform(t)
    assert torch.allclose(r0, t, atol=1e-3)
    r180 = RotateImageTransform(180.0, fixed=True).transform(t)
    assert torch.allclose(r180, t.flip(1, 2), atol=1e-2)
    assert torch.allclose(ColorConversionTransform("GRAY").transform(t)[0], 0.299 * t[0] + 0.587 * t[1] + 0.114 * t[2])
    hsv = ColorConversionTransform("HSV").transform(t)
    assert float(hsv[0, 0, 0]) == 0.0 and float(hsv[0, 0, -1]) == 120.0 and float(hsv[2, 0, -1]) == 200.0
    eq = EqualizeHistTransform().transform(torch.tensor([[[10.0, 10.0, 20.0, 30.0]]]))
    assert eq.reshape(-1).tolist() == [0.0, 0.0, 128.0, 255.0]
    assert tuple(BoxImageTransform(40, 10).transform(t).shape) == (3, 10, 40)
    pipe = PipelineImageTransform([(FlipImageTransform(1), 1.0), (CropImageTransform(1), 1.0), (FlipImageTransform(0), 0.0)])
    assert torch.equal(pipe.transform(t), t.flip(2)[:, 1:-1, 1:-1])
    flipped = NativeImageLoader(20, 30, 3, imageTransform=FlipImageTransform(1)).asMatrix(p)
    assert float(flipped[0, 0, 0, -1]) == 255.0
