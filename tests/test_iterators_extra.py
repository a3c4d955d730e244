"""The remaining utility iterators: adapters, file-backed, singleton / block / scrollable / joint, callbacks."""
import os

import pytest
import torch

from deeplearning4j_b200.data import (AsyncMultiDataSetIterator, BenchmarkMultiDataSetIterator, CombinedPreProcessor, DataSet, DataSetDeserializer,
                                      DataSetLoaderIterator, DoublesDataSetIterator, DummyBlockDataSetIterator, EarlyTerminationMultiDataSetIterator,
                                      FileDataSetIterator, FileMultiDataSetIterator, FileSplitDataSetIterator, FileSplitParallelDataSetIterator,
                                      FloatsDataSetIterator, InterleavedDataSetCallback, IteratorDataSetIterator, JointMultiDataSetIterator,
                                      ListDataSetIterator, MultiBoolean, MultiDataSet, MultiDataSetIteratorSplitter, RandomMultiDataSetIterator,
                                      ReconstructionDataSetIterator, ScrollableDataSetIterator, SingletonDataSetIterator, WorkspacesShieldDataSetIterator)


def _ds(n, seed=0, nin=3):
    g = torch.Generator().manual_seed(seed)
    return DataSet(torch.rand(n, nin, generator=g), torch.rand(n, 2, generator=g))


def test_adapters_and_rebatching():
    pairs = [([float(i), float(i) + 0.5], [float(i % 2)]) for i in range(7)]
    it = FloatsDataSetIterator(pairs, 3)
    sizes = [d.numExamples() for d in it]
    assert sizes == [3, 3, 1] and it.next if True else None
    it.reset()
    assert it.next().features.dtype == torch.float32 and DoublesDataSetIterator(pairs, 7).next().labels.dtype == torch.float64
    rb = IteratorDataSetIterator([_ds(5, 1), _ds(2, 2), _ds(6, 3)], 4)
    got = [d.numExamples() for d in rb]
    assert got == [4, 4, 4, 1]
    rb.reset()
    first = rb.next()
    assert torch.equal(first.features, _ds(5, 1).features[:4])
    one = SingletonDataSetIterator(_ds(3))
    assert [d.numExamples() for d in one] == [3] and not one.hasNext()
    one.reset()
    assert one.hasNext()
    blk = DummyBlockDataSetIterator(ListDataSetIterator([_ds(2, i) for i in range(5)]))
    assert len(blk.next(3)) == 3 and len(blk.next(3)) == 2
    rec = ReconstructionDataSetIterator(ListDataSetIterator([_ds(4)])).next()
    assert torch.equal(rec.features, rec.labels)
    sh = WorkspacesShieldDataSetIterator(ListDataSetIterator([_ds(4)])).next()
    assert torch.equal(sh.features, _ds(4).features)


def test_scrollable_splitter_joint_random_and_async():
    base = ListDataSetIterator([_ds(2, i) for i in range(10)])
    sp = MultiDataSetIteratorSplitter(base, 10, 0.7)
    tr = sp.getTrainIterator()
    assert len(list(tr)) == 7
    te = sp.getTestIterator()
    got = list(te)
    assert len(got) == 3 and torch.equal(got[0].features, _ds(2, 7).features)
    assert len(list(ScrollableDataSetIterator(0, base, ratio=0.5, totalBatches=10))) == 5
    j = JointMultiDataSetIterator(ListDataSetIterator([_ds(2, 1)]), ListDataSetIterator([_ds(2, 2, nin=5)]), outcome=1)
    m = j.next()
    assert isinstance(m, MultiDataSet) and [f.shape[1] for f in m.features] == [3, 5] and len(m.labels) == 1
    r = (RandomMultiDataSetIterator.Builder(3).addFeatures((4, 6), RandomMultiDataSetIterator.RANDOM_NORMAL)
         .addFeatures((4, 2), RandomMultiDataSetIterator.INTEGER_0_10).addLabels((4, 5), RandomMultiDataSetIterator.ONE_HOT).setSeed(7).build())
    ms = list(r)
    assert len(ms) == 3 and torch.equal(ms[0].labels[0].sum(1), torch.ones(4)) and float(ms[0].features[1].max()) < 10
    r.reset()
    assert torch.equal(r.next().features[0], ms[0].features[0])
    b = BenchmarkMultiDataSetIterator([(8, 3), (8, 4)], [5], 4)
    assert len(list(b)) == 4
    et = EarlyTerminationMultiDataSetIterator(r, 2)
    et.reset()
    assert len(list(et)) == 2
    with pytest.raises(ValueError):
        EarlyTerminationMultiDataSetIterator(r, 0)
    a = AsyncMultiDataSetIterator(ListDataSetIterator([_ds(2, i) for i in range(6)]), 2)
    assert len(list(a)) == 6
    a.reset()
    assert torch.equal(a.next().features, _ds(2, 0).features)
    a.shutdown()


def test_file_iterators_and_callbacks(tmp_path):
    d = tmp_path / "ds"
    d.mkdir()
    for i in range(4):
        _ds(3, i).save(str(d / f"part{i}.bin"))
    (d / "note.txt").write_text("x")
    it = FileDataSetIterator(str(d), validExtensions=["bin"])
    assert [x.numExamples() for x in it] == [3, 3, 3, 3]
    it2 = FileDataSetIterator(str(d), validExtensions=["bin"], batchSize=5)
    assert [x.numExamples() for x in it2] == [5, 5, 2]
    sh = FileDataSetIterator(str(d), validExtensions=["bin"], randomSeed=3)
    order_a = [float(x.features[0, 0]) for x in sh]
    sh.reset()
    assert order_a == [float(x.features[0, 0]) for x in sh] and sorted(order_a) == sorted(float(_ds(3, i).features[0, 0]) for i in range(4))
    md = tmp_path / "mds"
    md.mkdir()
    for i in range(3):
        MultiDataSet([torch.full((2, 2), float(i))], [torch.full((2, 1), float(i))]).save(str(md / f"m{i}.bin"))
    fm = FileMultiDataSetIterator(str(md), batchSize=3)
    assert [m.features[0].shape[0] for m in fm] == [3, 3]
    files = sorted(str(p) for p in d.glob("*.bin"))
    fs = FileSplitDataSetIterator(files, DataSetDeserializer())
    assert len(list(fs)) == 4
    par = FileSplitParallelDataSetIterator(str(d), "*.bin", DataSetDeserializer(), numThreads=2)
    assert len(list(par)) == 4
    ld = DataSetLoaderIterator(files, DataSet.load, shuffleSeed=1)
    assert len(list(ld)) == 4
    cb = InterleavedDataSetCallback([torch.device("cpu"), torch.device("cpu")])
    x = _ds(2)
    cb.call(x)
    cb.call(x)
    assert cb.k == 2
    calls = []

    class P:
        def __init__(s, k): s.k = k
        def preProcess(s, ds): calls.append(s.k)
    CombinedPreProcessor.Builder().addPreProcessor(1, P("b")).addPreProcessor(0, P("a")).build().preProcess(x)
    assert calls == ["a", "b"]
    mb = MultiBoolean(3)
    assert mb.allFalse() and not mb.allTrue()
    for i in range(3):
        mb.set(True, i)
    assert mb.allTrue()
    one = MultiBoolean(2, True, oneTime=True)
    one.set(False, 0)
    one.set(True, 0)
    assert not one.allTrue()
    with pytest.raises(ValueError):
        MultiBoolean(33)
