"""DataVec record readers, TransformProcess and the DataSet iterators built on them."""
import numpy as np
import pytest
import torch

from deeplearning4j_b200.datavec import (AlignmentMode, AnalyzeLocal, BooleanCondition, CollectionRecordReader, ColumnCondition, ConditionFilter,
                                         ConditionOp, CSVRecordReader, CSVSequenceRecordReader, FileSplit, ImageRecordReader, JacksonLineRecordReader,
                                         LocalTransformExecutor, MathOp, NumberedFileInputSplit, ParentPathLabelGenerator,
                                         RecordReaderDataSetIterator, Reducer, ReduceOp, RegexLineRecordReader, Schema,
                                         SequenceRecordReaderDataSetIterator, StringSplit, SVMLightRecordReader, TransformProcess,
                                         TransformProcessRecordReader)


def test_csv_reader_and_dataset_iterator(tmp_path):
    p = tmp_path / "iris.csv"
    rows = ["sl,sw,pl,pw,cls"] + [f"{5 + i * 0.1:.1f},{3.0},{1.4 + i},{0.2},{i % 3}" for i in range(10)] + ['"6,5",1,2,3,1']
    p.write_text("\n".join(rows) + "\n")
    rr = CSVRecordReader(1).initialize(FileSplit(str(p)))
    recs = list(rr)
    assert len(recs) == 11 and recs[0] == [5.0, 3.0, 1.4, 0.2, 0] and recs[-1][0] == "6,5"
    rr = CSVRecordReader(1).initialize(FileSplit(str(p)))
    it = RecordReaderDataSetIterator(rr, 4, 4, 3, maxNumBatches=2)
    batches = list(it)
    assert [tuple(b.getFeatures().shape) for b in batches] == [(4, 4), (4, 4)]
    assert batches[0].getLabels().tolist()[1] == [0.0, 1.0, 0.0] and it.inputColumns() == 4
    reg = RecordReaderDataSetIterator.Builder(CSVRecordReader(1).initialize(StringSplit("h\n1,2,3,4\n5,6,7,8")), 2).regression(2, 3).build().next()
    assert reg.getLabels().tolist() == [[3.0, 4.0], [7.0, 8.0]] and reg.getFeatures().tolist() == [[1.0, 2.0], [5.0, 6.0]]


def test_other_readers(tmp_path):
    rx = RegexLineRecordReader(r"(\d+)-(\w+) (.*)").initialize(StringSplit("12-ab hello world\n7-z x"))
    assert list(rx) == [[12, "ab", "hello world"], [7, "z", "x"]]
    js = JacksonLineRecordReader(["a", "b/c"]).initialize(StringSplit('{"a": 1, "b": {"c": "x"}}\n{"a": 2}'))
    assert list(js) == [[1, "x"], [2, None]]
    sv = SVMLightRecordReader(4).initialize(StringSplit("1 1:0.5 3:2\n0 2:1 # c"))
    assert list(sv) == [[0.5, 0.0, 2.0, 0.0, 1], [0.0, 1.0, 0.0, 0.0, 0]]
    for cls, val in (("cats", 10), ("dogs", 200)):
        d = tmp_path / "img" / cls
        d.mkdir(parents=True)
        for k in range(2):
            (d / f"{k}.ppm").write_bytes(b"P6\n4 2\n255\n" + bytes([val] * 24))
            np.save(d / f"{k}n.npy", np.full((3, 2, 4), float(val), dtype=np.float32))
    ir = ImageRecordReader(4, 4, 3, ParentPathLabelGenerator()).initialize(FileSplit(str(tmp_path / "img"), ["ppm", "npy"]))
    ds = RecordReaderDataSetIterator(ir, 8, 1, 2).next()
    assert tuple(ds.getFeatures().shape) == (8, 3, 4, 4) and ir.getLabels() == ["cats", "dogs"]
    assert ds.getLabels().sum(0).tolist() == [4.0, 4.0] and float(ds.getFeatures()[ds.getLabels()[:, 1] == 1].mean()) == 200.0


def test_sequence_iterator_alignment(tmp_path):
    for i, T in enumerate([3, 5]):
        (tmp_path / f"f_{i}.csv").write_text("\n".join(f"{t},{t * 2}" for t in range(T)))
        (tmp_path / f"l_{i}.csv").write_text("\n".join(str(t % 2) for t in range(T)))
    fr = CSVSequenceRecordReader().initialize(NumberedFileInputSplit(str(tmp_path / "f_%d.csv"), 0, 1))
    lr = CSVSequenceRecordReader().initialize(NumberedFileInputSplit(str(tmp_path / "l_%d.csv"), 0, 1))
    ds = SequenceRecordReaderDataSetIterator(fr, lr, 2, 2, alignmentMode=AlignmentMode.ALIGN_END).next()
    assert tuple(ds.getFeatures().shape) == (2, 2, 5) and ds.getFeaturesMaskArray().tolist() == [[0, 0, 1, 1, 1], [1, 1, 1, 1, 1]]
    assert ds.getFeatures()[0, :, 2:].tolist() == [[0, 1, 2], [0, 2, 4]] and ds.getLabels()[1, :, 1].tolist() == [0.0, 1.0]
    fr.reset(); lr.reset()
    with pytest.raises(ValueError):
        SequenceRecordReaderDataSetIterator(fr, lr, 2, 2, alignmentMode=AlignmentMode.EQUAL_LENGTH).next()


def test_transform_process_schema_filter_reduce_and_json():
    schema = (Schema.Builder().addColumnString("id").addColumnCategorical("color", "red", "green", "blue").addColumnDouble("price")
              .addColumnInteger("qty").build())
    tp = (TransformProcess.Builder(schema).filter(ConditionFilter(ColumnCondition("qty", ConditionOp.LessThan, 1)))
          .doubleMathOp("price", MathOp.Multiply, 2.0).doubleColumnsMathOp("total", MathOp.Multiply, "price", "qty")
          .conditionalReplaceValueTransform("total", 0.0, BooleanCondition.AND(ColumnCondition("color", ConditionOp.Equal, "blue"),
                                                                             ColumnCondition("qty", ConditionOp.GreaterThan, 5)))
          .categoricalToOneHot("color").removeColumns("id").renameColumn("qty", "quantity").build())
    assert tp.getFinalSchema().getColumnNames() == ["color[red]", "color[green]", "color[blue]", "price", "quantity", "total"]
    recs = [["a", "red", 1.5, 2], ["b", "blue", 1.0, 0], ["c", "blue", 2.0, 10], ["d", "green", 3.0, 1]]
    out = LocalTransformExecutor.execute(recs, tp)
    assert out == [[1, 0, 0, 3.0, 2, 6.0], [0, 0, 1, 4.0, 10, 0.0], [0, 1, 0, 6.0, 1, 6.0]]
    tp2 = TransformProcess.fromJson(tp.toJson())
    assert LocalTransformExecutor.execute(recs, tp2) == out and tp2.getFinalSchema() == tp.getFinalSchema()
    rr = TransformProcessRecordReader(CollectionRecordReader(recs), tp).initialize(None)
    assert RecordReaderDataSetIterator(rr, 10, 5, 1, regression=True).next().getFeatures().shape == (3, 5)
    red = (TransformProcess.Builder(schema).removeColumns("id")
           .reduce(Reducer.Builder(ReduceOp.Sum).keyColumns("color").meanColumns("price").countColumns("qty").build()).build())
    assert red.getFinalSchema().getColumnNames() == ["color", "mean(price)", "count(qty)"]
    assert LocalTransformExecutor.execute(recs, red) == [["red", 1.5, 1], ["blue", 1.5, 2], ["green", 3.0, 1]]
    seq = TransformProcess.Builder(schema).convertToSequence("color", "qty").build()
    s = LocalTransformExecutor.execute(recs, seq)
    assert [len(x) for x in s] == [1, 2, 1] and [r[3] for r in s[1]] == [0, 10]
    an = AnalyzeLocal.analyze(schema, recs)
    assert an.getColumnAnalysis("price")["max"] == 3.0 and an.getColumnAnalysis("color")["mapOfCounts"]["blue"] == 2
