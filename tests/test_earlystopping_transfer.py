"""Early stopping and transfer learning on small CPU networks."""
import pytest
import torch

from deeplearning4j_b200 import nn
from deeplearning4j_b200.data.dataset import DataSet
from deeplearning4j_b200.data.iterators import ListDataSetIterator
from deeplearning4j_b200.nn.earlystopping import (DataSetLossCalculator, EarlyStoppingConfiguration, EarlyStoppingTrainer, InMemoryModelSaver,
                                                  InvalidScoreIterationTerminationCondition, LocalFileModelSaver, MaxEpochsTerminationCondition,
                                                  MaxScoreIterationTerminationCondition, ScoreImprovementEpochTerminationCondition,
                                                  ClassificationScoreCalculator, TerminationReason)
from deeplearning4j_b200.nn.transferlearning import FineTuneConfiguration, TransferLearning, TransferLearningHelper


def _net(lr=5e-2, nout=3):
    conf = (nn.NeuralNetConfiguration.Builder().seed(7).updater(nn.Adam(lr)).list()
            .layer(nn.DenseLayer(nIn=4, nOut=16, activation="tanh"))
            .layer(nn.DenseLayer(nIn=16, nOut=8, activation="tanh"))
            .layer(nn.OutputLayer("MCXENT", nIn=8, nOut=nout, activation="softmax")).build())
    return nn.MultiLayerNetwork(conf).init()


def _iter(n=6, batch=32, seed=0, classes=3):
    g = torch.Generator().manual_seed(seed)
    sets = []
    for _ in range(n):
        x = torch.randn(batch, 4, generator=g)
        y = ((x[:, 0] > 0).long() + (x[:, 1] > 0).long()) % classes
        sets.append(DataSet(x, torch.nn.functional.one_hot(y, classes).float()))
    return ListDataSetIterator(sets)


def test_early_stopping_max_epochs_and_best_model(tmp_path):
    saver = LocalFileModelSaver(str(tmp_path))
    es = (EarlyStoppingConfiguration.Builder().epochTerminationConditions(MaxEpochsTerminationCondition(6))
          .iterationTerminationConditions(InvalidScoreIterationTerminationCondition())
          .scoreCalculator(DataSetLossCalculator(_iter(2, seed=9), True)).modelSaver(saver).saveLastModel(True).build())
    net = _net()
    res = EarlyStoppingTrainer(es, net, _iter()).fit()
    assert res.getTerminationReason() == TerminationReason.EpochTerminationCondition and res.getTotalEpochs() == 6
    assert len(res.getScoreVsEpoch()) == 6 and res.getBestModelScore() == min(res.getScoreVsEpoch().values())
    best = res.getBestModel()
    assert best is not None and abs(DataSetLossCalculator(_iter(2, seed=9)).calculateScore(best) - res.getBestModelScore()) < 1e-5
    assert saver.getLatestModel() is not None


def test_early_stopping_no_improvement_and_iteration_condition():
    es = (EarlyStoppingConfiguration.Builder()
          .epochTerminationConditions(MaxEpochsTerminationCondition(200), ScoreImprovementEpochTerminationCondition(2, 10.0))
          .scoreCalculator(ClassificationScoreCalculator("ACCURACY", _iter(2, seed=9))).modelSaver(InMemoryModelSaver()).build())
    res = EarlyStoppingTrainer(es, _net(), _iter()).fit()
    assert res.getTotalEpochs() == 3 and "ScoreImprovement" in res.getTerminationDetails()       # accuracy cannot improve by 10
    es = (EarlyStoppingConfiguration.Builder().epochTerminationConditions(MaxEpochsTerminationCondition(5))
          .iterationTerminationConditions(MaxScoreIterationTerminationCondition(1e-9)).build())
    res = EarlyStoppingTrainer(es, _net(), _iter()).fit()
    assert res.getTerminationReason() == TerminationReason.IterationTerminationCondition and res.getTotalEpochs() == 0


def test_transfer_learning_freeze_replace_and_add():
    src = _net()
    src.fit(_iter(), 3)
    ftc = FineTuneConfiguration.builder().updater(nn.Sgd(0.1)).build()
    net = (TransferLearning.Builder(src).fineTuneConfiguration(ftc).setFeatureExtractor(0)
           .nOutReplace(1, 12, "XAVIER").removeOutputLayer()
           .addLayer(nn.OutputLayer("MCXENT", nIn=12, nOut=2, activation="softmax")).build())
    assert net.getnLayers() == 3 and type(net.conf.layers()[0]).__name__ == "FrozenLayer"
    p_src, p_new = src.paramTable(), net.paramTable()
    assert torch.equal(p_src["0_W"].t, p_new["0_W"].t) and tuple(p_new["1_W"].t.shape) == (16, 12) and tuple(p_new["2_W"].t.shape) == (12, 2)
    w0 = p_new["0_W"].t.clone()
    w1 = p_new["1_W"].t.clone()
    net.fit(_iter(classes=2), 2)
    assert torch.equal(net.paramTable()["0_W"].t, w0)               # frozen layer did not move
    assert not torch.equal(net.paramTable()["1_W"].t, w1)
    assert type(net.conf.layers()[1].updater).__name__ == "Sgd"


def test_transfer_learning_helper_featurize():
    src = _net()
    helper = TransferLearningHelper(src, 0)
    ds = next(iter(_iter(1)))
    feat = helper.featurize(ds)
    assert tuple(feat.getFeatures().shape) == (32, 16)
    before = helper.net.paramTable()["1_W"].t.clone()
    out_a = helper.net.output(ds.getFeatures())
    out_b = helper.outputFromFeaturized(feat.getFeatures())
    assert torch.allclose(out_a.t, out_b.t, atol=1e-6)
    for _ in range(3):
        helper.fitFeaturized(feat)
    assert not torch.equal(helper.net.paramTable()["1_W"].t, before)
    assert torch.allclose(helper.net.output(ds.getFeatures()).t, helper.outputFromFeaturized(feat.getFeatures()).t, atol=1e-6)


def test_transfer_learning_graph():
    g = (nn.NeuralNetConfiguration.Builder().seed(3).updater(nn.Adam(1e-2)).graphBuilder().addInputs("in")
         .addLayer("d0", nn.DenseLayer(nIn=4, nOut=10, activation="relu"), "in")
         .addLayer("d1", nn.DenseLayer(nIn=10, nOut=6, activation="relu"), "d0")
         .addLayer("out", nn.OutputLayer("MCXENT", nIn=6, nOut=3, activation="softmax"), "d1").setOutputs("out").build())
    from deeplearning4j_b200.nn.graph import ComputationGraph
    cg = ComputationGraph(g).init()
    new = (TransferLearning.GraphBuilder(cg).setFeatureExtractor("d0").removeVertexAndConnections("out")
           .addLayer("out2", nn.OutputLayer("MCXENT", nIn=6, nOut=2, activation="softmax"), "d1").setOutputs("out2").build())
    assert torch.equal(cg.paramTable()["d0_W"].t, new.paramTable()["d0_W"].t) and torch.equal(cg.paramTable()["d1_W"].t, new.paramTable()["d1_W"].t)
    w0 = new.paramTable()["d0_W"].t.clone()
    it = _iter(classes=2)
    new.fit(it, 2)
    assert torch.equal(new.paramTable()["d0_W"].t, w0) and tuple(new.paramTable()["out2_W"].t.shape) == (6, 2)
