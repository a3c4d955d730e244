"""Evaluation classes against hand-computed values and scikit-learn."""
import numpy as np
import pytest
import torch
from sklearn import metrics as skm

from deeplearning4j_b200.eval import (ROC, Evaluation, EvaluationBinary, EvaluationCalibration, EvaluationTools, RegressionEvaluation,
                                      ROCBinary, ROCMultiClass)


def _data(n=400, c=4, seed=0):
    g = torch.Generator().manual_seed(seed)
    y = torch.randint(0, c, (n,), generator=g)
    logits = torch.randn(n, c, generator=g) + 2.0 * torch.nn.functional.one_hot(y, c)
    return torch.nn.functional.one_hot(y, c).float(), logits.softmax(1), y


def test_evaluation_matches_sklearn_macro():
    lab, p, y = _data()
    e = Evaluation()
    e.eval(lab[:150], p[:150])
    e2 = Evaluation()
    e2.eval(lab[150:], p[150:])
    e.merge(e2)
    pred = p.argmax(1).numpy()
    assert e.accuracy() == pytest.approx(skm.accuracy_score(y, pred))
    assert e.precision() == pytest.approx(skm.precision_score(y, pred, average="macro"))
    assert e.recall() == pytest.approx(skm.recall_score(y, pred, average="macro"))
    assert e.f1() == pytest.approx(skm.f1_score(y, pred, average="macro"))
    assert e.precision(averaging="Micro") == pytest.approx(skm.precision_score(y, pred, average="micro"))
    assert np.array_equal(e.confusionMatrix().numpy(), skm.confusion_matrix(y, pred))
    assert e.matthewsCorrelation(2) == pytest.approx(skm.matthews_corrcoef(y == 2, pred == 2))
    assert "Accuracy" in e.stats() and Evaluation.fromJson(e.toJson()).f1() == e.f1()


def test_evaluation_binary_positive_class_topn_and_time_series():
    lab, p, y = _data(c=2, seed=3)
    e = Evaluation()
    e.eval(lab, p)
    pred = p.argmax(1).numpy()
    assert e.precision() == pytest.approx(skm.precision_score(y, pred))          # positive class only
    assert e.f1() == pytest.approx(skm.f1_score(y, pred))
    lab, p, y = _data(c=5, seed=4)
    e = Evaluation(topN=3)
    e.eval(lab, p)
    assert e.topNAccuracy() == pytest.approx(skm.top_k_accuracy_score(y, p.numpy(), k=3))
    # [N,C,T] with a mask: masked steps must not count
    l3, p3 = lab[:40].reshape(4, 10, 5).permute(0, 2, 1), p[:40].reshape(4, 10, 5).permute(0, 2, 1)
    mask = torch.ones(4, 10)
    mask[:, 7:] = 0
    e = Evaluation()
    e.eval(l3, p3, mask)
    assert e.getNumRowCounter() == 28


def test_roc_exact_and_thresholded_match_sklearn():
    g = torch.Generator().manual_seed(1)
    y = (torch.rand(500, generator=g) > 0.6).float()
    p = (torch.rand(500, generator=g) * 0.6 + 0.4 * y * torch.rand(500, generator=g)).clamp(0, 1)
    r = ROC(0)
    r.eval(y[:200, None], p[:200, None])
    r.eval(y[200:, None], p[200:, None])
    assert r.calculateAUC() == pytest.approx(skm.roc_auc_score(y, p), abs=1e-9)
    pr, rc, _ = skm.precision_recall_curve(y, p)
    assert r.calculateAUCPR() == pytest.approx(skm.auc(rc, pr), abs=2e-3)
    rt = ROC(200)
    rt.eval(y[:, None], p[:, None])
    assert rt.calculateAUC() == pytest.approx(skm.roc_auc_score(y, p), abs=5e-3)
    assert r.getRocCurve().calculateAUC() == pytest.approx(r.calculateAUC(), abs=1e-9)
    assert "<svg" in EvaluationTools.rocChartToHtml(r)


def test_roc_multiclass_binary_and_evaluation_binary():
    lab, p, y = _data(c=3, seed=5)
    rm = ROCMultiClass(0)
    rm.eval(lab, p)
    for c in range(3):
        assert rm.calculateAUC(c) == pytest.approx(skm.roc_auc_score(y == c, p[:, c]), abs=1e-9)
    g = torch.Generator().manual_seed(2)
    yb = (torch.rand(300, 3, generator=g) > 0.5).float()
    pb = (yb * 0.3 + torch.rand(300, 3, generator=g) * 0.7)
    rb = ROCBinary(0)
    rb.eval(yb, pb)
    assert rb.calculateAUC(1) == pytest.approx(skm.roc_auc_score(yb[:, 1], pb[:, 1]), abs=1e-9)
    eb = EvaluationBinary()
    eb.eval(yb, pb)
    for c in range(3):
        assert eb.accuracy(c) == pytest.approx(skm.accuracy_score(yb[:, c], pb[:, c] > 0.5))
        assert eb.f1(c) == pytest.approx(skm.f1_score(yb[:, c], pb[:, c] > 0.5))
    assert "label_0" in eb.stats()


def test_regression_and_calibration():
    g = torch.Generator().manual_seed(7)
    y = torch.randn(200, 3, generator=g)
    p = y + 0.3 * torch.randn(200, 3, generator=g)
    r = RegressionEvaluation()
    r.eval(y[:90], p[:90])
    r.eval(y[90:], p[90:])
    for c in range(3):
        assert r.meanSquaredError(c) == pytest.approx(skm.mean_squared_error(y[:, c], p[:, c]))
        assert r.meanAbsoluteError(c) == pytest.approx(skm.mean_absolute_error(y[:, c], p[:, c]))
        assert r.rSquared(c) == pytest.approx(skm.r2_score(y[:, c], p[:, c]))
        assert r.pearsonCorrelation(c) == pytest.approx(np.corrcoef(y[:, c], p[:, c])[0, 1])
    assert "MSE" in r.stats()
    lab, pr, _ = _data(c=3, seed=9)
    ec = EvaluationCalibration(10, 20)
    ec.eval(lab, pr)
    d = ec.getReliabilityDiagram(0)
    assert len(d["meanPredictedValueX"]) == len(d["fractionPositivesY"]) > 0
    assert sum(ec.getLabelCountsEachClass()) == 400 and sum(ec.getProbabilityHistogramAllClasses()["binCounts"]) == 1200
    assert 0 <= ec.expectedCalibrationError(1) < 0.3
