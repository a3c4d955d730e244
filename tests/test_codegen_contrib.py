"""Op DSL -> generated namespaces / docs, and the contrib analyzers."""
import os

import pytest
import torch

from deeplearning4j_b200.codegen.dsl import BOOL, FLOATING_POINT, INT, NUMERIC, Arg, Constraint, Input, NamespaceDef, Output
from deeplearning4j_b200.contrib import analyzers


def _ns():
    ns = NamespaceDef("demo")
    ns.Op("abs", inputs=[Input("x", NUMERIC, "input array")], doc="Element-wise absolute value.")
    ns.Op("clipByValue", libnd4jName="clipbyvalue", inputs=[Input("x", NUMERIC)],
          args=[Arg("clipValueMin", FLOATING_POINT, "lower bound", -1.0), Arg("clipValueMax", FLOATING_POINT, "upper bound", 1.0)],
          doc="Clips to [min, max].", constraints=[Constraint("min must not exceed max", lambda a: a["clipValueMin"] <= a["clipValueMax"])])
    ns.Op("sum", libnd4jName="reduce_sum", inputs=[Input("x", NUMERIC)], args=[Arg("keepDims", BOOL, default=False), Arg("dimensions", INT, count="N")],
          outputs=[Output("output", NUMERIC, "reduced array")], doc="Sum over dimensions.")
    return ns.validate()


def test_dsl_generates_working_namespaces_and_docs():
    ns = _ns()
    g = {}
    exec(ns.generatePython("ND"), g)
    nd = g["NDDemo"]()
    from deeplearning4j_b200 import Nd4j
    x = Nd4j.create([[-2.0, 0.5], [3.0, -0.25]])
    assert nd.abs(x).t.tolist() == [[2.0, 0.5], [3.0, 0.25]]
    assert nd.clipByValue(x, clipValueMin=-1.0, clipValueMax=1.0).t.tolist() == [[-1.0, 0.5], [1.0, -0.25]]
    assert nd.sum(x, keepDims=True, dimensions=[1]).t.tolist() == [[-1.5], [2.75]]
    exec(ns.generatePython("SD"), g)
    from deeplearning4j_b200.samediff.core import SameDiff
    sd = SameDiff.create()
    v = sd.var("v", torch.tensor([-1.0, 2.0]))
    out = g["SDDemo"](sd).abs("a", v)
    assert out.name == "a" and sd.output({}, "a")["a"].t.tolist() == [1.0, 2.0]
    docs = ns.generateDocs()
    assert "## clipByValue" in docs and "native op `clipbyvalue`" in docs and "**clipValueMin** (FLOATING_POINT, default -1.0)" in docs
    assert '"libnd4jName": "reduce_sum"' in ns.toJson()
    assert ns.check("clipByValue", clipValueMin=2.0, clipValueMax=1.0) == ["min must not exceed max"] and not ns.check("clipByValue", clipValueMin=0.0, clipValueMax=1.0)
    with pytest.raises(ValueError, match="not in the op registry"):
        NamespaceDef("bad", []).Op("nope_nope").validate()
    bad = NamespaceDef("bad2")
    bad.Op("abs", inputs=[Input("x")])
    bad.Op("abs", inputs=[Input("x")])
    with pytest.raises(ValueError, match="defined twice"):
        bad.validate()


def test_profiler_launch_list_analyzer(tmp_path):
    p = tmp_path / "launches.csv"
    p.write_text('==PROF== Connected to process 1\n"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"\n'
                 '"0","1","python","h","void dl4j::gemm_tcgen05_kernel<256, 0, 1>(CUtensorMap_st, GemmParams)","1","7","(192, 1, 1)","(148, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","ns","60,000"\n'
                 '"1","1","python","h","dl4j::fused_update_kernel(float *, float *)","1","7","(256, 1, 1)","(100, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","ns","30000"\n'
                 '"2","1","python","h","void dl4j::gemm_tcgen05_kernel<128, 0, 0>(CUtensorMap_st, GemmParams)","1","7","(192, 1, 1)","(148, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","ns","10000"\n')
    rows = analyzers.kernel_shares(str(p))
    assert [r["kernel"] for r in rows] == ["dl4j::gemm_tcgen05_kernel", "dl4j::fused_update_kernel"] and rows[0]["launches"] == 2
    assert abs(rows[0]["ms"] - 0.07) < 1e-9 and abs(rows[0]["share"] - 0.7) < 1e-9
    assert "| 70.0 % | 0.070 ms | 2 | dl4j::gemm_tcgen05_kernel |" in analyzers.shares_markdown(rows)
    assert analyzers.step_boundaries(str(p)) == [1]


def test_native_dependency_analyzer_and_registry_report():
    src = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "deeplearning4j_b200", "csrc")
    deps = analyzers.native_dependencies(src)
    assert "common.cuh" in deps["gemm_tcgen05.cu"]["includes"] and "dl4j_gemm" in deps["gemm_tcgen05.cu"]["exports"]
    assert "flash_common.cuh" in deps["flash_attn_fwd.cu"]["includes"] and "common.cuh" in deps["flash_attn_fwd.cu"]["includes"]
    assert "w2v_batch_kernel" in deps["nlp_kernels.cu"]["kernels"]
    assert analyzers.rebuild_set(src, "flash_common.cuh") == ["flash_attn_bwd.cu", "flash_attn_fwd.cu"]
    assert len(analyzers.rebuild_set(src, "common.cuh")) >= 10
    rep = analyzers.registry_report()
    assert rep["missing"] == [] and rep["registered"] >= 519
