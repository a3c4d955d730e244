"""FlatGraph files written by the reference (classic shapeInfo arrays, legacy op numbers, positional op arguments, logic nodes) and
graph-level control flow built here (``ifCond`` / ``whileLoop`` as enter / merge / switch / exit / next_iteration nodes).

Golden values are the ones the reference's own tests state for these files
(``libnd4j/tests_cpu/layers_tests/ConditionalTests.cpp:248-320``, ``OneOffTests.cpp:96-260``)."""
import glob
import os

import pytest
import torch

from deeplearning4j_b200 import DataType
from deeplearning4j_b200.samediff.controlflow import DataflowExecutor, has_logic_ops
from deeplearning4j_b200.samediff.core import SameDiff
from deeplearning4j_b200.samediff.serde.flatgraph import Utf8Array, from_flatbuffers, to_flatbuffers

_RES = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "reference", "libnd4j", "tests_cpu", "resources")
_FILES = sorted(glob.glob(os.path.join(_RES, "*.fb")))
needs_fixtures = pytest.mark.skipif(len(_FILES) < 20, reason="the reference's FlatGraph fixtures are not available next to this checkout")


def _load(name):
    with open(os.path.join(_RES, name), "rb") as f:
        return from_flatbuffers(f.read())


def _run(sd, ph=None):
    feeds = dict(ph or {})
    for n, v in sd.variables.items():
        if v.variableType == "PLACEHOLDER" and n not in sd.arrays and n not in feeds:
            feeds[n] = torch.ones([int(s) for s in (v._shape or [])])
    return DataflowExecutor(sd).run(feeds)


@needs_fixtures
def test_every_reference_fixture_loads_and_executes():
    assert len(_FILES) == 20
    for f in _FILES:
        sd = from_flatbuffers(open(f, "rb").read())
        assert sd.ops, f
        vals = _run(sd)
        produced = [o for n in sd.ops for o in n.outputs if o in vals]
        assert produced, f


@needs_fixtures
def test_shape_info_arrays_big_endian_and_strings():
    sd = _load("avg_pooling3d.fb")
    x = sd.arrays["in_0"]
    assert tuple(x.shape) == (1, 2, 5, 5, 5) and x.dtype == torch.float32
    assert 0.0 <= float(x.min()) and float(x.max()) <= 1.0          # big-endian floats decoded, not byte-swapped garbage
    sd = _load("assertsomething.fb")
    msg = sd.arrays["assert_equal/Assert/AssertGuard/Assert/data_0"]
    assert isinstance(msg, Utf8Array) and len(msg) == 1 and isinstance(msg[0], str)
    sd = _load("non2d_1.fb")
    assert sd.arrays["Reshape/shape"].numel() == 0                   # empty array flag in the shapeInfo extras


@needs_fixtures
@pytest.mark.parametrize("x0,expected", [(-4.0, -1.0), (-9.0, -3.0)])
def test_while_loop_fixture_matches_reference_values(x0, expected):
    sd = _load("simplewhile_1.fb")
    assert has_logic_ops(sd)
    vals = _run(sd, {"input_0": torch.full((2, 2), x0), "input_1": torch.tensor(1.0)})
    assert torch.equal(vals["output"], torch.full((2, 2), expected))


@needs_fixtures
def test_nested_while_and_conditional_fixtures():
    vals = _run(_load("simplewhile_nested.fb"))
    assert torch.equal(vals["output"], torch.full((2, 2), 15.0))
    sd = _load("simpleif_0_alt.fb")
    v_true = _run(sd, {"input_0": torch.full((2, 2), 1.0), "input_1": torch.tensor(5.0)})
    v_false = _run(sd, {"input_0": torch.full((2, 2), 1.0), "input_1": torch.tensor(-5.0)})
    assert torch.equal(v_true["output"], torch.full((2, 2), 3.0))          # sum(x) < y: x + Variable
    assert torch.equal(v_false["output"], torch.full((2, 2), -1.0))        # else: x - Variable
    assert "cond/falsefn" not in v_true and "cond/truefn" not in v_false   # the untaken branch computed nothing
    vals = _run(_load("cond_true.fb"))
    assert torch.equal(vals["cond/Merge"], torch.ones(5))


@needs_fixtures
def test_legacy_and_positional_argument_nodes():
    vals = _run(_load("pad_1D.fb"))
    exp = torch.tensor([10.0, 0.778786, 0.801198, 0.724375, 0.230894, 0.727141, 10.0])
    torch.testing.assert_close(vals["PadV2"], exp, atol=1e-5, rtol=1e-5)
    vals = _run(_load("channels_last_b1_k2_s1_d1_SAME_crelu.fb"))
    z = vals["conv2d/CRelu/Relu"]
    assert tuple(z.shape) == (1, 5, 5, 6)
    torch.testing.assert_close(z[0, 0, 0], torch.tensor([0.55744928, 0.76827729, 1.09401524, 0.0, 0.0, 0.0]), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(z[0, 4, 4], torch.tensor([0.17486368, 0.44460732, 0.44499981, 0.0, 0.0, 0.0]), atol=1e-5, rtol=1e-5)
    vals = _run(_load("reduce_all_rank2_d0_keep.fb"))
    assert tuple(vals["All"].shape) == (1, 4) and vals["All"].dtype == torch.bool
    vals = _run(_load("tensor_array_close_sz1_float32_nodynamic_noname_noshape.fb"))
    exp = torch.tensor([[0.77878559, 0.80119777, 0.72437465], [0.23089433, 0.72714126, 0.18039072]])
    torch.testing.assert_close(vals["TensorArrayReadV3"], exp, atol=1e-6, rtol=1e-6)


def test_legacy_op_table_resolves_to_registered_ops():
    from deeplearning4j_b200.ops import registry
    from deeplearning4j_b200.samediff.serde.legacy_ops import LEGACY_OPS
    assert LEGACY_OPS["REDUCE_SAME"][0] == ("Sum", "reduce_sum")
    assert LEGACY_OPS["TRANSFORM_SAME"][3][0] == "Neg" and LEGACY_OPS["SCALAR"][39][0] == "RELU"
    total = sum(len(v) for v in LEGACY_OPS.values())
    missing = [(f, n, v) for f, ops in LEGACY_OPS.items() for n, v in ops.items() if not registry.has(v[1])]
    assert total >= 300 and not missing, missing[:5]


# ------------------------------------------------------------------------------------------------- control flow built here
def _while_graph():
    sd = SameDiff.create()
    x = sd.placeHolder("x", DataType.FLOAT, 2, 2)
    lim = sd.var("lim", torch.tensor(10.0))
    start = sd._op("identity", [x])
    cond = lambda s, v: s._op("less", [s._op("reduce_sum", [v[0]]), lim])
    body = lambda s, v: [s._op("add", [v[0], s.constant(None, torch.tensor(1.0))]), s._op("add", [v[1], v[0]])]
    outs = sd.whileLoop([start, start], cond, body)
    return sd, outs


def test_while_loop_is_graph_nodes_and_survives_fb_round_trip():
    sd, outs = _while_graph()
    names = {o.opName for o in sd.ops}
    assert {"enter", "merge", "loop_cond", "switch", "exit", "next_iteration"} <= names
    r = sd.output({"x": torch.zeros(2, 2)}, outs[0].name, outs[1].name)
    assert torch.equal(r[outs[0].name].toTorch(), torch.full((2, 2), 3.0))       # 4 * i >= 10 first at i = 3
    assert torch.equal(r[outs[1].name].toTorch(), torch.full((2, 2), 3.0))       # 0 + 0 + 1 + 2
    sd2 = from_flatbuffers(to_flatbuffers(sd))
    r2 = sd2.output({"x": torch.zeros(2, 2)}, outs[0].name, outs[1].name)
    assert torch.equal(r2[outs[0].name].toTorch(), r[outs[0].name].toTorch())
    assert torch.equal(r2[outs[1].name].toTorch(), r[outs[1].name].toTorch())
    r3 = sd2.output({"x": torch.full((2, 2), 5.0)}, outs[0].name)
    assert torch.equal(r3[outs[0].name].toTorch(), torch.full((2, 2), 5.0))      # condition false at once: zero iterations


def test_if_cond_runs_only_the_taken_branch_and_round_trips():
    sd = SameDiff.create()
    a = sd.placeHolder("a", DataType.FLOAT, 2)
    b = sd.var("b", torch.tensor([1.0, 5.0]))
    aa = sd._op("identity", [a])
    res = sd.ifCond(lambda s: s._op("less", [s._op("reduce_sum", [aa]), s.constant(None, torch.tensor(0.0))]),
                    lambda s: s._op("add", [aa, b], name="taken_if_negative"), lambda s: s._op("subtract", [aa, b], name="taken_otherwise"))
    for sdx in (sd, from_flatbuffers(to_flatbuffers(sd))):
        neg = DataflowExecutor(sdx).run({"a": torch.tensor([-1.0, -2.0])})
        pos = DataflowExecutor(sdx).run({"a": torch.tensor([1.0, 2.0])})
        assert torch.equal(neg[res.name], torch.tensor([0.0, 3.0])) and "taken_otherwise" not in neg
        assert torch.equal(pos[res.name], torch.tensor([0.0, -3.0])) and "taken_if_negative" not in pos


def test_gradient_flows_through_a_graph_loop():
    sd = SameDiff.create()
    w = sd.var("w", torch.tensor(2.0))
    x = sd.placeHolder("x", DataType.FLOAT)
    start = sd._op("identity", [x])
    cnt = sd._op("identity", [sd.constant(None, torch.tensor(0.0))])
    o = sd.whileLoop([start, cnt], lambda s, v: s._op("less", [v[1], s.constant(None, torch.tensor(3.0))]),
                     lambda s, v: [s._op("multiply", [v[0], w]), s._op("add", [v[1], s.constant(None, torch.tensor(1.0))])])
    sd.setLossVariables(o[0].name)
    g = sd.calculateGradients({"x": torch.tensor(1.5)}, "w")
    assert abs(float(g["w"].toTorch()) - 18.0) < 1e-5                             # d/dw (x w^3) = 3 x w^2


def test_nested_graph_loops():
    sd = SameDiff.create()
    x = sd.placeHolder("x", DataType.FLOAT)
    i0 = sd._op("identity", [x])
    acc0 = sd._op("identity", [sd.constant(None, torch.tensor(0.0))])
    one = lambda s: s.constant(None, torch.tensor(1.0))

    def outer_body(s, v):
        j0 = s._op("identity", [s.constant(None, torch.tensor(0.0))])
        inner = s.whileLoop([j0, v[1]], lambda s2, u: s2._op("less", [u[0], s2.constant(None, torch.tensor(2.0))]),
                            lambda s2, u: [s2._op("add", [u[0], one(s2)]), s2._op("add", [u[1], v[0]])])
        return [s._op("add", [v[0], one(s)]), inner[1]]
    o = sd.whileLoop([i0, acc0], lambda s, v: s._op("less", [v[0], s.constant(None, torch.tensor(3.0))]), outer_body)
    r = sd.output({"x": torch.tensor(0.0)}, o[1].name)
    assert float(r[o[1].name].toTorch()) == 2 * (0 + 1 + 2)                      # inner loop adds i twice for i = 0, 1, 2
