"""ONNX import: models are encoded with the bundled protobuf writer (no onnx package) and checked against torch."""
import numpy as np
import torch
import torch.nn.functional as F

from deeplearning4j_b200.importers import protowire as pw
from deeplearning4j_b200.importers.onnx_import import OnnxFrameworkImporter, parse_model


def tensor(name, arr):
    arr = np.ascontiguousarray(arr)
    dt = {np.dtype("float32"): 1, np.dtype("int64"): 7}[arr.dtype]
    return pw.field_packed_varints(1, arr.shape) + pw.field_varint(2, dt) + pw.field_string(8, name) + pw.field_bytes(9, arr.tobytes())


def attr(name, v):
    b = pw.field_string(1, name)
    if isinstance(v, float):
        return b + pw.field_float(2, v) + pw.field_varint(20, 1)
    if isinstance(v, int):
        return b + pw.field_varint(3, v) + pw.field_varint(20, 2)
    if isinstance(v, str):
        return b + pw.field_bytes(4, v.encode()) + pw.field_varint(20, 3)
    if isinstance(v, (list, tuple)):
        return b + pw.field_packed_varints(8, v) + pw.field_varint(20, 7)
    raise TypeError(v)


def node(op, ins, outs, **attrs):
    b = b"".join(pw.field_string(1, i) for i in ins) + b"".join(pw.field_string(2, o) for o in outs) + pw.field_string(3, outs[0] + "_node") + pw.field_string(4, op)
    return b + b"".join(pw.field_bytes(5, attr(k, v)) for k, v in attrs.items())


def value_info(name, shape):
    dims = b"".join(pw.field_bytes(1, pw.field_varint(1, d)) for d in shape)
    tt = pw.field_varint(1, 1) + pw.field_bytes(2, dims)
    return pw.field_string(1, name) + pw.field_bytes(2, pw.field_bytes(1, tt))


def model(nodes, inits, inputs, outputs):
    g = b"".join(pw.field_bytes(1, n) for n in nodes) + pw.field_string(2, "g") + b"".join(pw.field_bytes(5, t) for t in inits)
    g += b"".join(pw.field_bytes(11, value_info(n, s)) for n, s in inputs) + b"".join(pw.field_bytes(12, value_info(n, s)) for n, s in outputs)
    return pw.field_varint(1, 8) + pw.field_bytes(7, g) + pw.field_bytes(8, pw.field_string(1, "") + pw.field_varint(2, 13))


def test_cnn_graph_matches_torch(tmp_path):
    g = torch.Generator().manual_seed(0)
    W = torch.randn(4, 3, 3, 3, generator=g) * 0.3
    b = torch.randn(4, generator=g) * 0.1
    sc, bi, mu, var = torch.rand(4, generator=g) + 0.5, torch.randn(4, generator=g), torch.randn(4, generator=g) * 0.1, torch.rand(4, generator=g) + 0.5
    Wd = torch.randn(5, 4 * 4 * 4, generator=g) * 0.1
    bd = torch.randn(5, generator=g) * 0.1
    nodes = [node("Conv", ["x", "W", "b"], ["c"], kernel_shape=[3, 3], pads=[1, 1, 1, 1], strides=[1, 1]),
             node("BatchNormalization", ["c", "sc", "bi", "mu", "var"], ["bn"], epsilon=1e-5), node("Relu", ["bn"], ["r"]),
             node("MaxPool", ["r"], ["p"], kernel_shape=[2, 2], strides=[2, 2]), node("Flatten", ["p"], ["f"], axis=1),
             node("Gemm", ["f", "Wd", "bd"], ["logits"], transB=1), node("Softmax", ["logits"], ["prob"], axis=1)]
    inits = [tensor(n, t.numpy()) for n, t in (("W", W), ("b", b), ("sc", sc), ("bi", bi), ("mu", mu), ("var", var), ("Wd", Wd), ("bd", bd))]
    raw = model(nodes, inits, [("x", [1, 3, 8, 8])], [("prob", [1, 5])])
    parsed = parse_model(raw)
    assert [n["op"] for n in parsed["nodes"]][:2] == ["Conv", "BatchNormalization"] and parsed["nodes"][0]["attrs"]["pads"] == [1, 1, 1, 1] and parsed["opset"] == 13
    p = tmp_path / "m.onnx"
    p.write_bytes(raw)
    imp = OnnxFrameworkImporter()
    sd = imp.runImport(str(p))
    x = torch.randn(2, 3, 8, 8, generator=g)
    got = sd.output({"x": x}, "prob")["prob"].t
    ref = F.conv2d(x, W, b, padding=1)
    ref = F.batch_norm(ref, mu, var, sc, bi, False, 0.0, 1e-5)
    ref = F.softmax(F.linear(F.max_pool2d(F.relu(ref), 2).flatten(1), Wd, bd), 1)
    assert torch.allclose(got, ref, atol=1e-5) and imp.outputs == ["prob"]
    assert {"W", "Wd"} <= {v.name for v in sd.trainableVariables()}


def test_elementwise_shape_ops_and_unsupported():
    shp = np.asarray([2, -1], dtype=np.int64)
    nodes = [node("Reshape", ["x", "shape"], ["r"]), node("Transpose", ["r"], ["t"], perm=[1, 0]), node("ReduceMean", ["t"], ["m"], axes=[0], keepdims=0),
             node("Mul", ["m", "m"], ["sq"]), node("Concat", ["sq", "m"], ["cat"], axis=0), node("Unsqueeze", ["cat"], ["u"], axes=[0]),
             node("Clip", ["u"], ["out"], min=-0.5, max=0.5)]
    raw = model(nodes, [tensor("shape", shp)], [("x", [12])], [("out", [1, 4])])
    sd = OnnxFrameworkImporter().runImport(raw)
    x = torch.arange(12.0) / 10 - 0.5
    got = sd.output({"x": x}, "out")["out"].t
    m = x.reshape(2, 6).t().mean(0)
    assert torch.allclose(got, torch.cat([m * m, m]).unsqueeze(0).clamp(-0.5, 0.5), atol=1e-6)
    bad = model([node("NonMaxSuppressionXYZ", ["x"], ["y"])], [], [("x", [1])], [("y", [1])])
    try:
        OnnxFrameworkImporter().runImport(bad)
        assert False
    except NotImplementedError as e:
        assert "NonMaxSuppressionXYZ" in str(e)
