"""Training listeners (DL4J and SameDiff flavours), checkpoints and host-side failure injection."""
import io
import json
import os

import pytest
import torch

from deeplearning4j_b200 import nn
from deeplearning4j_b200.data.dataset import DataSet
from deeplearning4j_b200.data.iterators import ListDataSetIterator
from deeplearning4j_b200.listeners import (CallType, CheckpointListener, CollectScoresListener, EvaluativeListener, FailureMode,
                                           FailureTestingListener, InvocationType, IterationEpochTrigger, PerformanceListener,
                                           ScoreIterationListener, TimeIterationListener)


def _net():
    conf = (nn.NeuralNetConfiguration.Builder().seed(1).updater(nn.Adam(1e-2)).list()
            .layer(nn.DenseLayer(nIn=4, nOut=8, activation="relu"))
            .layer(nn.OutputLayer("MCXENT", nIn=8, nOut=3, activation="softmax")).build())
    return nn.MultiLayerNetwork(conf).init()


def _iter(n=8, batch=16):
    g = torch.Generator().manual_seed(0)
    sets = []
    for _ in range(n):
        x = torch.randn(batch, 4, generator=g)
        y = torch.nn.functional.one_hot((x[:, 0] > 0).long() + (x[:, 1] > 0).long(), 3).float()
        sets.append(DataSet(x, y))
    return ListDataSetIterator(sets)


def test_score_performance_collect_time_listeners():
    net = _net()
    out = io.StringIO()
    perf = PerformanceListener(2, reportScore=True, out=out)
    coll = CollectScoresListener(1)
    tl = TimeIterationListener(16)
    net.setListeners(ScoreIterationListener(4, out=out), perf, coll, tl)
    net.fit(_iter(), 2)
    text = out.getvalue()
    assert "Score at iteration 0 is" in text and "samples/sec:" in text and "batches/sec:" in text and "ETL:" in text
    assert coll.getListIteration() == list(range(16)) and coll.getListScore()[-1] < coll.getListScore()[0]
    assert perf.samplesPerSec > 0 and "Remaining time" in tl.lastMessage


def test_checkpoint_listener_keep_last_and_restore(tmp_path):
    net = _net()
    cl = CheckpointListener.builder(str(tmp_path)).saveEveryNIterations(3).keepLast(2).build()
    net.setListeners(cl)
    net.fit(_iter(), 2)
    zips = sorted(f for f in os.listdir(tmp_path) if f.endswith(".zip"))
    assert len(zips) == 2 and all(z.startswith("checkpoint_") and z.endswith("_MultiLayerNetwork.zip") for z in zips)
    lines = open(tmp_path / "checkpointInfo.txt").read().splitlines()
    assert lines[0] == "checkpointNum,timestamp,iteration,epoch,modelType,filename" and len(lines) == 6
    avail = CheckpointListener.availableCheckpoints(str(tmp_path))
    assert [c.checkpointNum for c in avail] == [3, 4]
    restored = CheckpointListener.loadLastCheckpointMLN(str(tmp_path))
    assert restored.getIterationCount() == avail[-1].iteration + 1 or restored.getIterationCount() == avail[-1].iteration
    with pytest.raises(ValueError):
        CheckpointListener.builder(str(tmp_path)).saveEveryEpoch().build()          # directory already has checkpoints
    with pytest.raises(ValueError):
        CheckpointListener.builder(str(tmp_path / "x")).build()                      # no schedule


def test_evaluative_listener_and_failure_injection():
    net = _net()
    ev = EvaluativeListener(_iter(2), 1, InvocationType.EPOCH_END)
    net.setListeners(ev)
    net.fit(_iter(), 3)
    assert ev.invocationCount == 3 and ev.getEvaluations()[0].accuracy() > 0.4
    net = _net()
    net.setListeners(FailureTestingListener(FailureMode.ILLEGAL_STATE, IterationEpochTrigger(False, 5)))
    with pytest.raises(RuntimeError, match="FailureTestingListener"):
        net.fit(_iter(), 1)
    net = _net()
    net.setListeners(FailureTestingListener(FailureMode.OOM, IterationEpochTrigger(True, 1)))
    with pytest.raises(MemoryError):
        net.fit(_iter(), 3)
    assert net.getEpochCount() == 1
    slept = FailureTestingListener(FailureMode.INFINITE_SLEEP, IterationEpochTrigger(False, 0), sleepSeconds=0.1)
    slept.iterationDone(net, 0, 0)


def test_samediff_listeners(tmp_path):
    from deeplearning4j_b200 import DataType
    from deeplearning4j_b200.samediff.core import SameDiff
    from deeplearning4j_b200.samediff.listeners import (ArraySavingListener, CheckpointListener as SDCheckpoint, ExecDebuggingListener,
                                                        HistoryListener, OpBenchmarkListener, ProfilingListener, ScoreListener, UIListener)
    from deeplearning4j_b200.samediff.training import TrainingConfig
    sd = SameDiff.create()
    x = sd.placeHolder("x", DataType.FLOAT, -1, 4)
    y = sd.placeHolder("y", DataType.FLOAT, -1, 3)
    w = sd.var("w", torch.randn(4, 3) * 0.1)
    b = sd.var("b", torch.zeros(3))
    logits = sd.nn.linear(x, w, b)
    loss = sd.loss.softmaxCrossEntropy("loss", y, logits)
    sd.setLossVariables("loss")
    sd.setTrainingConfig(TrainingConfig.builder().updater(nn.Adam(1e-2)).dataSetFeatureMapping("x").dataSetLabelMapping("y").build())
    out = io.StringIO()
    prof = ProfilingListener(str(tmp_path / "trace.json"))
    hist, bench, dbg = HistoryListener(), OpBenchmarkListener(), ExecDebuggingListener("SHAPES_ONLY", out=out)
    ck = SDCheckpoint.builder(str(tmp_path / "ck")).saveEveryNEpochs(1).keepLast(1).build()
    sd.setListeners(ScoreListener(2, out=out), hist, prof, bench, dbg, ArraySavingListener(str(tmp_path / "arr")),
                    UIListener(str(tmp_path / "ui.log")), ck)
    sd.fit(_iter(4), 2)
    prof.close()
    trace = json.load(open(tmp_path / "trace.json"))
    assert trace["traceEvents"] and {"name", "ph", "ts", "dur", "pid", "tid"} <= set(trace["traceEvents"][0])
    assert "Loss at epoch 0, iteration 0" in out.getvalue() and "shapes=" in out.getvalue()
    assert len(hist.getReport()["lossCurve"]) == 2 and len(hist.getReport()["lossCurve"][0]) == 4
    assert any(v["count"] >= 8 for v in bench.getAggregateModeMap().values()) and "ms/call" in bench.printTimings()
    assert any(f.endswith(".npy") for f in os.listdir(tmp_path / "arr"))
    recs = [json.loads(l) for l in open(tmp_path / "ui.log")]
    assert recs[0]["type"] == "graph" and sum(r["type"] == "loss" for r in recs) == 8
    assert len([f for f in os.listdir(tmp_path / "ck") if f.startswith("checkpoint-")]) == 1
    sd2 = ck.loadLast()
    assert torch.equal(sd2.arrays["w"], sd.arrays["w"].cpu())
