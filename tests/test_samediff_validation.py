"""SameDiff GradCheckUtil / OpValidation over a sample of ops (the reference's opvalidation suites)."""
import math

import torch

from deeplearning4j_b200 import DataType
from deeplearning4j_b200.samediff.core import SameDiff
from deeplearning4j_b200.samediff.validation import GradCheckUtil, OpTestCase, OpValidation, TestCase


def test_graph_gradients_match_numerical():
    sd = SameDiff.create()
    g = torch.Generator().manual_seed(0)
    x = sd.placeHolder("x", DataType.DOUBLE, -1, 4)
    y = sd.placeHolder("y", DataType.DOUBLE, -1, 3)
    w1 = sd.var("w1", torch.randn(4, 6, generator=g, dtype=torch.float64) * 0.5)
    b1 = sd.var("b1", torch.randn(6, generator=g, dtype=torch.float64) * 0.1)
    gam = sd.var("gam", torch.rand(6, generator=g, dtype=torch.float64) + 0.5)
    bet = sd.var("bet", torch.zeros(6, dtype=torch.float64))
    w2 = sd.var("w2", torch.randn(6, 3, generator=g, dtype=torch.float64) * 0.5)
    h = sd.nn.layerNorm(sd.nn.tanh(x.mmul(w1).add(b1)), gam, bet, False, 1)
    h = sd.math.square(h).add(sd.nn.softplus(h))
    loss = sd.loss.softmaxCrossEntropy("loss", y, h.mmul(w2))
    sd.setLossVariables("loss")
    ph = {"x": torch.randn(5, 4, generator=g, dtype=torch.float64), "y": torch.nn.functional.one_hot(torch.randint(0, 3, (5,), generator=g), 3).double()}
    assert GradCheckUtil.checkGradients(sd, ph, print_=False)
    tc = TestCase(sd).testName("mlp").placeholderValues(ph).expectedOutput("loss", lambda t: True if t.numel() == 1 else "not scalar")
    assert OpValidation.validate(tc) is None
    bad = TestCase(sd).placeholderValues(ph).expectedOutput("loss", torch.tensor(123.0)).gradientCheck(False)
    assert "differs" in OpValidation.validate(bad)


def test_single_op_cases_and_coverage():
    x = torch.tensor([[1.0, -2.0, 3.0], [0.5, 0.0, -1.0]])
    cases = [OpTestCase("add", [x, x]).expectedOutput(0, 2 * x), OpTestCase("reduce_sum", [x], dimensions=[1]).expectedOutput(0, x.sum(1)),
             OpTestCase("softmax", [x]).expectedOutput(0, torch.softmax(x, -1)), OpTestCase("transpose", [x]).expectedOutputShape(0, (3, 2)),
             OpTestCase("gelu", [x]).expectedOutput(0, x * torch.sigmoid(1.702 * x)), OpTestCase("precise_gelu", [x]).expectedOutput(0, torch.nn.functional.gelu(x, approximate="tanh")),
             OpTestCase("matmul", [x, x.t()]).expectedOutput(0, x @ x.t()), OpTestCase("argmax", [x], dimensions=[1]).expectedOutput(0, x.argmax(1)),
             OpTestCase("cumsum", [x], dimensions=[1]).expectedOutput(0, x.cumsum(1)), OpTestCase("tile", [x], reps=[2, 1]).expectedOutputShape(0, (4, 3))]
    for c in cases:
        assert OpValidation.validate(c) is None, c.opName
    assert "differs" in OpValidation.validate(OpTestCase("add", [x, x]).expectedOutput(0, x))
    cov = OpValidation.coverage()
    assert cov["validated"] >= 10 and cov["total"] > 500 and "Op validation coverage" in OpValidation.logCoverageInformation()


def test_graph_optimizer_folds_constants_removes_identities_and_unused_ops():
    import numpy as np
    from deeplearning4j_b200 import DataType, Nd4j
    from deeplearning4j_b200.samediff import SameDiff
    from deeplearning4j_b200.samediff.optimize import GraphOptimizer
    sd = SameDiff.create()
    x = sd.placeHolder("x", DataType.FLOAT, -1, 3)
    c1 = sd.constant("c1", Nd4j.create([1.0, 2.0, 3.0]))
    c2 = sd.constant("c2", Nd4j.create([10.0, 20.0, 30.0]))
    folded = c1.mul(c2).add(c1)                       # constants only: becomes one constant
    y = x.add(0.0).mul(1.0)                          # identities
    y = sd.math.neg(sd.math.neg(y))
    out = y.add(folded).rename("out")
    unused = sd.math.exp(x).rename("unused")          # does not reach the output
    n_before = len(sd.ops)
    opt = GraphOptimizer.optimize(sd, "out")
    assert len(opt.ops) == 1 and opt.ops[0].opName == "add" and len(sd.ops) == n_before      # original untouched
    assert "unused" not in opt.variables
    xv = np.random.default_rng(0).normal(size=(4, 3)).astype(np.float32)
    a = sd.output({"x": Nd4j.create(xv)}, "out")["out"].numpy()
    b = opt.output({"x": Nd4j.create(xv)}, "out")["out"].numpy()
    np.testing.assert_allclose(a, b, rtol=1e-6)
    np.testing.assert_allclose(b, xv + np.array([11.0, 42.0, 93.0], dtype=np.float32), rtol=1e-6)


def test_op_log_listener_finds_first_divergence(tmp_path):
    import numpy as np
    from deeplearning4j_b200 import DataType, Nd4j
    from deeplearning4j_b200.contrib import OpLogAnalyzer, OpLogListener
    from deeplearning4j_b200.samediff import SameDiff

    def build(scale):
        sd = SameDiff.create()
        x = sd.placeHolder("x", DataType.FLOAT, -1, 3)
        w = sd.var("w", Nd4j.create(np.eye(3, dtype=np.float32) * scale))
        h = x.mmul(w).rename("h")
        sd.math.tanh(h).rename("t").sum().rename("s")
        return sd
    xv = Nd4j.create(np.arange(6, dtype=np.float32).reshape(2, 3))
    paths = []
    for i, scale in enumerate((1.0, 1.0, 1.5)):
        p = str(tmp_path / f"log{i}.db")
        sd = build(scale)
        lst = OpLogListener(p)
        sd.addListeners(lst)
        sd.output({"x": xv}, "s")
        lst.close()
        paths.append(p)
    same = OpLogAnalyzer.compare(paths[0], paths[1])
    assert same["first_divergence"] is None and not same["missing_in_b"]
    diff = OpLogAnalyzer.compare(paths[0], paths[2])
    assert diff["first_divergence"]["op"] in ("matmul", "mmul") and len(diff["diverged"]) == 3
    assert {op for op, n, ms in OpLogAnalyzer.summary(paths[0])} >= {"tanh", "reduce_sum"}


def test_ops_benchmark_suite_runs_on_cpu():
    from deeplearning4j_b200.bench import ops_suite
    rows = ops_suite.run("light", "cpu", filt="transform/exp", iters=2, warmup=1)
    assert len(rows) == 2 and all(r["ms"] > 0 and r["gbs"] > 0 for r in rows)
    rows = ops_suite.run("light", "cpu", filt="blas/matmul", iters=1, warmup=1)
    assert rows and "gflops" in rows[0]
