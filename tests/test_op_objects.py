"""DynamicCustomOp / OpContext / OpExecutioner / user-defined ops, and SameDiff eager mode."""
import pytest
import torch

from deeplearning4j_b200 import Nd4j
from deeplearning4j_b200.ops.executioner import DynamicCustomOp, OpContext, OpExecutioner, ProfilingMode, UserDefinedCustomOp
from deeplearning4j_b200.samediff.core import SameDiff


def test_dynamic_custom_op_with_positional_arguments():
    x = Nd4j.create([[1.0, 2, 3], [4, 5, 6]])
    op = DynamicCustomOp.builder("reduce_sum").addInputs(x).addIntegerArguments(1).addBooleanArguments(True).build()
    out = Nd4j.exec(op)
    assert out[0].t.tolist() == [[6.0], [15.0]] and op.getOutputArgument(0).t.tolist() == [[6.0], [15.0]]
    assert op.opName() == "reduce_sum" and op.iArgs() == [1] and op.bArgs() == [True] and op.numInputArguments() == 1
    assert op.calculateOutputShape()[0]["shape"] == (2, 1)
    # conv2d reads kH, kW, sH, sW, pH, pW, dH, dW, isSameMode, dataFormat, wFormat as integers
    img, w = Nd4j.rand(1, 2, 5, 5), Nd4j.rand(3, 2, 3, 3)
    conv = DynamicCustomOp.builder("conv2d").addInputs(img, w).addIntegerArguments(3, 3, 1, 1, 0, 0, 1, 1, 0, 0, 1).build()
    y = Nd4j.exec(conv)[0]
    assert torch.allclose(y.t, torch.nn.functional.conv2d(img.t, w.t), atol=1e-5)
    # preallocated output and in-place call
    dst = Nd4j.zeros(2, 3)
    Nd4j.exec(DynamicCustomOp.builder("add").addInputs(x, x).addOutputs(dst).build())
    assert dst.t.tolist() == [[2, 4, 6], [8, 10, 12]]
    z = Nd4j.create([-1.0, 2.0])
    Nd4j.exec(DynamicCustomOp.builder("relu").addInputs(z).addFloatingPointArguments(0.0).callInplace(True).build())
    assert z.t.tolist() == [0.0, 2.0]
    with pytest.raises(KeyError):
        DynamicCustomOp.builder("no_such_op").build()


def test_op_context_and_executioner_modes():
    ex = Nd4j.getExecutioner()
    assert ex is OpExecutioner.instance() and ex.type() in ("CUDA", "NATIVE_CPU")
    op = DynamicCustomOp.builder("softmax").build()
    ctx = ex.buildContext()
    ctx.setInputArrays(Nd4j.create([[1.0, 2.0, 3.0]]))
    ctx.setIArguments(1)
    out = ex.exec(op, ctx)
    assert torch.allclose(out[0].t, torch.softmax(torch.tensor([[1.0, 2.0, 3.0]]), 1)) and ctx.getOutputArray(0) is not None
    ex.setProfilingMode(ProfilingMode.NAN_PANIC)
    try:
        with pytest.raises(FloatingPointError):
            ex.exec("log", Nd4j.create([-1.0]))
        ex.setProfilingMode(ProfilingMode.OPERATIONS)
        ex.exec("exp", Nd4j.create([0.0]))
        assert ex.stats["exp"][0] >= 1 and ex.getLastOp() == "exp"
    finally:
        ex.setProfilingMode(ProfilingMode.DISABLED)
    assert "torch" in ex.getEnvironmentInformation()
    ex.commit()


class Swish2(UserDefinedCustomOp):
    def exec(self, inputs):
        x, = inputs
        return [x * torch.sigmoid(2 * x)]

    def doDiff(self, inputs, outputs, gradients):
        x, = inputs
        s = torch.sigmoid(2 * x)
        return [gradients[0] * (s + 2 * x * s * (1 - s))]


def test_user_defined_op_in_a_graph_with_its_own_gradient():
    sd = SameDiff.create()
    x = sd.var("x", torch.tensor([0.5, -1.0, 2.0]))
    y = sd.doUdf(Swish2(), x, name="y")
    loss = sd.math.sum(y) if hasattr(sd.math, "sum") else sd._op("reduce_sum", [y])
    sd.setLossVariables(loss.name)
    out = sd.output({}, "y")["y"].t
    xt = torch.tensor([0.5, -1.0, 2.0], requires_grad=True)
    ref = xt * torch.sigmoid(2 * xt)
    assert torch.allclose(out, ref.detach())
    g = sd.calculateGradients({}, "x")["x"].t
    ref.sum().backward()
    assert torch.allclose(g, xt.grad, atol=1e-6)
    assert Nd4j.exec(Swish2(), Nd4j.create([1.0]))[0].t.item() == pytest.approx(float(torch.sigmoid(torch.tensor(2.0))))


def test_eager_mode_gives_arrays_while_the_graph_is_defined():
    sd = SameDiff.create().enableEagerMode()
    a = sd.var("a", torch.tensor([1.0, 2.0]))
    b = sd.constant("b", torch.tensor([10.0, 20.0]))
    c = a.add(b) if hasattr(a, "add") else sd._op("add", [a, b])
    assert sd.isEagerMode() and c.getArr().t.tolist() == [11.0, 22.0]
    p = sd.placeHolder("p", None, 2)
    d = sd._op("multiply", [c, p])
    assert d.getArr() is None                                  # depends on a placeholder: stays symbolic
    assert sd.output({"p": torch.tensor([2.0, 2.0])}, d.name)[d.name].t.tolist() == [22.0, 44.0]
