"""SameDiff define-then-run graphs: variables / placeholders / constants, namespaces, execution, autodiff against
torch.autograd, control flow, training with TrainingConfig.  Mirrors the intent of nd4j's SameDiffTests and
SameDiffTrainingTest."""
import numpy as np
import pytest
import torch

from deeplearning4j_b200 import DataType, Nd4j
from deeplearning4j_b200.samediff import SameDiff, TrainingConfig
from deeplearning4j_b200 import nn as dl4j_nn


def _t(a):
    return a.t if hasattr(a, "t") and isinstance(a.t, torch.Tensor) else torch.as_tensor(np.asarray(a))


def test_variables_placeholders_constants_and_exec():
    sd = SameDiff.create()
    x = sd.placeHolder("x", DataType.FLOAT, -1, 4)
    w = sd.var("w", Nd4j.create(np.arange(12, dtype=np.float32).reshape(4, 3) / 10))
    b = sd.constant("b", Nd4j.create([1.0, 2.0, 3.0]))
    y = x.mmul(w).add(b).rename("y")
    assert x.isPlaceHolder() and b.isConstant() and not w.isConstant()
    assert sd.hasVariable("y") and "w" in [v.name_() for v in sd.trainableVariables()]
    xv = np.ones((2, 4), dtype=np.float32)
    out = sd.output({"x": Nd4j.create(xv)}, "y")["y"]
    ref = xv @ (np.arange(12, dtype=np.float32).reshape(4, 3) / 10) + np.array([1, 2, 3], dtype=np.float32)
    np.testing.assert_allclose(out.numpy(), ref, rtol=1e-6)
    # eval on a variable-only subgraph needs no placeholders
    z = w.mul(2.0).sum()
    assert abs(float(z.eval().numpy()) - 2 * 6.6) < 1e-4


def test_gradients_match_torch_autograd():
    rng = np.random.default_rng(0)
    xv = rng.normal(size=(5, 4)).astype(np.float32)
    wv = rng.normal(size=(4, 3)).astype(np.float32)
    bv = rng.normal(size=(3,)).astype(np.float32)
    lab = np.eye(3, dtype=np.float32)[rng.integers(0, 3, size=5)]
    sd = SameDiff.create()
    x = sd.placeHolder("x", DataType.FLOAT, -1, 4)
    labels = sd.placeHolder("labels", DataType.FLOAT, -1, 3)
    w = sd.var("w", Nd4j.create(wv))
    b = sd.var("b", Nd4j.create(bv))
    h = sd.nn.tanh(x.mmul(w).add(b))
    loss = sd.loss.softmaxCrossEntropy("loss", labels, h, None)
    sd.setLossVariables("loss")
    grads = sd.calculateGradients({"x": Nd4j.create(xv), "labels": Nd4j.create(lab)}, "w", "b")
    tw, tb = torch.tensor(wv, requires_grad=True), torch.tensor(bv, requires_grad=True)
    logits = torch.tanh(torch.tensor(xv) @ tw + tb)
    ref = -(torch.tensor(lab) * torch.log_softmax(logits, -1)).sum(-1).mean()
    ref.backward()
    np.testing.assert_allclose(grads["w"].numpy(), tw.grad.numpy(), rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(grads["b"].numpy(), tb.grad.numpy(), rtol=1e-4, atol=1e-6)


def test_math_and_reduction_namespace_ops():
    sd = SameDiff.create()
    a = sd.var("a", Nd4j.create(np.array([[1.0, -2.0, 3.0], [4.0, 5.0, -6.0]], dtype=np.float32)))
    assert sd.math.abs(a).eval().numpy().tolist() == [[1, 2, 3], [4, 5, 6]]
    np.testing.assert_allclose(sd.math.exp(a).eval().numpy(), np.exp(a.getArr().numpy()), rtol=1e-6)
    np.testing.assert_allclose(a.sum(1).eval().numpy(), [2.0, 3.0])
    np.testing.assert_allclose(a.mean(0).eval().numpy(), [2.5, 1.5, -1.5])
    np.testing.assert_allclose(a.norm2(1).eval().numpy(), np.sqrt([14.0, 77.0]), rtol=1e-6)
    assert a.argmax(1).eval().numpy().tolist() == [2, 1]
    assert a.reshape(3, 2).eval().shape() == (3, 2)
    assert a.permute(1, 0).eval().shape() == (3, 2)
    sm = sd.nn.softmax(a, 1).eval().numpy()
    np.testing.assert_allclose(sm.sum(1), [1.0, 1.0], rtol=1e-6)
    ln = sd.nn.layerNorm(a, sd.constant("g", Nd4j.ones(3)), sd.constant("beta", Nd4j.zeros(3)), True, 1).eval().numpy()
    np.testing.assert_allclose(ln.mean(1), [0.0, 0.0], atol=1e-6)


def test_name_scopes_and_rename():
    sd = SameDiff.create()
    with sd.withNameScope("block"):
        v = sd.var("w", Nd4j.ones(2, 2))
        with sd.withNameScope("inner"):
            u = sd.var("w", Nd4j.ones(2, 2))
    assert v.name_() == "block/w" and u.name_() == "block/inner/w"
    sd.renameVariable("block/w", "renamed")
    assert sd.hasVariable("renamed") and not sd.hasVariable("block/w")


def test_control_flow_if_and_while():
    sd = SameDiff.create()
    x = sd.placeHolder("x", DataType.FLOAT)
    out = sd.ifCond("res", None, lambda s: x.gt(0.0), lambda s: x.mul(2.0), lambda s: x.neg())
    assert float(sd.output({"x": Nd4j.scalar(3.0)}, "res")["res"].numpy()) == 6.0
    assert float(sd.output({"x": Nd4j.scalar(-3.0)}, "res")["res"].numpy()) == 3.0
    sd2 = SameDiff.create()
    i0 = sd2.constant("i0", Nd4j.scalar(0.0))
    acc0 = sd2.constant("acc0", Nd4j.scalar(1.0))
    outs = sd2.whileLoop(["i", "acc"], None, [i0, acc0], lambda s, v: v[0].lt(5.0), lambda s, v: [v[0].add(1.0), v[1].mul(2.0)])
    res = sd2.output({}, outs[1].name_())[outs[1].name_()]
    assert float(res.numpy()) == 32.0


def test_training_reduces_loss_and_updates_variables():
    rng = np.random.default_rng(3)
    xv = rng.normal(size=(64, 5)).astype(np.float32)
    true_w = rng.normal(size=(5, 1)).astype(np.float32)
    yv = xv @ true_w
    sd = SameDiff.create()
    x = sd.placeHolder("x", DataType.FLOAT, -1, 5)
    y = sd.placeHolder("y", DataType.FLOAT, -1, 1)
    w = sd.var("w", Nd4j.zeros(5, 1))
    pred = x.mmul(w)
    sd.loss.meanSquaredError("loss", y, pred, None)
    sd.setLossVariables("loss")
    sd.setTrainingConfig(TrainingConfig.builder().updater(dl4j_nn.Adam(0.05)).dataSetFeatureMapping("x")
                         .dataSetLabelMapping("y").build())
    from deeplearning4j_b200.data import DataSet
    ds = DataSet(Nd4j.create(xv), Nd4j.create(yv))
    first = None
    for _ in range(150):
        h = sd.fit(ds)
        if first is None:
            first = float(sd.output({"x": ds.getFeatures(), "y": ds.getLabels()}, "loss")["loss"].numpy())
    last = float(sd.output({"x": ds.getFeatures(), "y": ds.getLabels()}, "loss")["loss"].numpy())
    assert last < 0.05 * first
    np.testing.assert_allclose(sd.getVariable("w").getArr().numpy(), true_w, atol=0.15)


def test_convert_constant_variable_and_dup():
    sd = SameDiff.create()
    w = sd.var("w", Nd4j.ones(2, 2))
    sd.convertToConstant(w)
    assert sd.getVariable("w").isConstant() and not sd.trainableVariables()
    sd.convertToVariable(sd.getVariable("w"))
    assert len(sd.trainableVariables()) == 1
    c = sd.dup()
    c.getVariable("w").getArr().addi(1.0)
    assert float(sd.getVariable("w").getArr().sumNumber()) == 4.0


def test_execution_trace_is_collected_into_a_graph():
    from deeplearning4j_b200.ops import registry
    Nd4j.purgeTrace()
    Nd4j.toggleTrace(True)
    try:
        a = torch.tensor([[1.0, -2.0], [3.0, 4.0]])
        b = registry.execute("abs", [a])
        c = registry.execute("matmul", [b, a], transposeY=True)
        d = registry.execute("reduce_sum", [c], dimensions=[1])
    finally:
        Nd4j.toggleTrace(False)
    traces = Nd4j.listTraces()
    assert [t.opName for t in traces] == ["abs", "matmul", "reduce_sum"] and traces[1].args == {"transposeY": True}
    sd = SameDiff.collectTrace()
    assert [o.opName for o in sd.ops] == ["abs", "matmul", "reduce_sum"]
    out = sd.output({}, sd.ops[-1].outputs[0])[sd.ops[-1].outputs[0]]
    np.testing.assert_allclose(out.numpy(), d.numpy())
    registry.execute("abs", [a])
    assert len(Nd4j.listTraces()) == 3                   # tracing is off again
    Nd4j.purgeTrace()
    assert not Nd4j.listTraces()


def test_residual_add_followed_by_layer_norm_runs_as_one_fused_node():
    from deeplearning4j_b200.samediff.session import _build_plan
    sd = SameDiff.create()
    x = sd.placeHolder("x", DataType.FLOAT, -1, 8)
    y = sd.placeHolder("y", DataType.FLOAT, -1, 8)
    gv, bv = np.linspace(0.5, 1.5, 8).astype(np.float32), np.linspace(-1, 1, 8).astype(np.float32)
    g, b = sd.var("g", Nd4j.create(gv)), sd.var("b", Nd4j.create(bv))
    h = sd.nn.layerNorm("ln", x.add(y), g, b, False, 1)
    loss = h.mul(h).sum().rename("loss")
    sd.setLossVariables("loss")
    assert [n.opName for n, _ in _build_plan(sd, ["loss"])] == ["add_layer_norm", "multiply", "reduce_sum"]
    # the sum itself requested as an output: no fusion
    s_name = sd.getVariable("ln").name_()
    add_out = [o.outputs[0] for o in sd.ops if o.opName == "add"][0]
    assert "add" in [n.opName for n, _ in _build_plan(sd, ["loss", add_out])]
    rng = np.random.default_rng(0)
    xv, yv = rng.normal(size=(4, 8)).astype(np.float32), rng.normal(size=(4, 8)).astype(np.float32)
    out = sd.output({"x": Nd4j.create(xv), "y": Nd4j.create(yv)}, "ln")["ln"].numpy()
    tx, ty = torch.tensor(xv, requires_grad=True), torch.tensor(yv)
    tg, tb = torch.tensor(gv, requires_grad=True), torch.tensor(bv, requires_grad=True)
    ref = torch.nn.functional.layer_norm(tx + ty, (8,), tg, tb, 1e-5)
    np.testing.assert_allclose(out, ref.detach().numpy(), rtol=1e-5, atol=1e-6)
    (ref * ref).sum().backward()
    grads = sd.calculateGradients({"x": Nd4j.create(xv), "y": Nd4j.create(yv)}, "g", "b")
    np.testing.assert_allclose(grads["g"].numpy(), tg.grad.numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(grads["b"].numpy(), tb.grad.numpy(), rtol=1e-4, atol=1e-5)
    # broadcasting operands keep the two-op semantics inside the fused node
    sd2 = SameDiff.create()
    a = sd2.placeHolder("a", DataType.FLOAT, -1, 8)
    p = sd2.constant("p", Nd4j.create(bv))
    sd2.nn.layerNorm("ln", a.add(p), sd2.constant("g", Nd4j.create(gv)), sd2.constant("b", Nd4j.create(bv)), False, 1)
    out2 = sd2.output({"a": Nd4j.create(xv)}, "ln")["ln"].numpy()
    ref2 = torch.nn.functional.layer_norm(torch.tensor(xv) + torch.tensor(bv), (8,), torch.tensor(gv), torch.tensor(bv), 1e-5)
    np.testing.assert_allclose(out2, ref2.numpy(), rtol=1e-5, atol=1e-6)
