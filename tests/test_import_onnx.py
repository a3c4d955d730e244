"""ONNX import: models are encoded with the bundled protobuf writer (no onnx package) and checked against torch."""
import numpy as np
import pytest
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
    if isinstance(v, bytes):                              # an encoded GraphProto
        return b + pw.field_bytes(6, v) + pw.field_varint(20, 5)
    raise TypeError(v)


def node(op, ins, outs, **attrs):
    b = b"".join(pw.field_string(1, i) for i in ins) + b"".join(pw.field_string(2, o) for o in outs) + pw.field_string(3, outs[0] + "_node") + pw.field_string(4, op)
    return b + b"".join(pw.field_bytes(5, attr(k, v)) for k, v in attrs.items())


def value_info(name, shape):
    dims = b"".join(pw.field_bytes(1, pw.field_varint(1, d)) for d in shape)
    tt = pw.field_varint(1, 1) + pw.field_bytes(2, dims)
    return pw.field_string(1, name) + pw.field_bytes(2, pw.field_bytes(1, tt))


def graph(nodes, inits, inputs, outputs):
    g = b"".join(pw.field_bytes(1, n) for n in nodes) + pw.field_string(2, "g") + b"".join(pw.field_bytes(5, t) for t in inits)
    return g + b"".join(pw.field_bytes(11, value_info(n, s)) for n, s in inputs) + b"".join(pw.field_bytes(12, value_info(n, s)) for n, s in outputs)


def model(nodes, inits, inputs, outputs):
    g = graph(nodes, inits, inputs, outputs)
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


def test_generic_rules_against_torch():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(2, 4, 6, 6, generator=g)
    Wt = torch.randn(4, 3, 3, 3, generator=g) * 0.2
    i64 = np.int64
    nodes = [
        node("Less", ["x", "zero"], ["lt"]), node("Where", ["lt", "zero", "x"], ["relu_like"]),
        node("ReduceL2", ["x"], ["l2"], axes=[1], keepdims=0), node("ReduceLogSumExp", ["x", "ax23"], ["lse"], keepdims=1),
        node("TopK", ["x", "k"], ["tv", "ti"], axis=3, largest=1), node("Split", ["x", "sizes"], ["s0", "s1"], axis=1),
        node("Pad", ["x", "pads"], ["pd"], mode="reflect"), node("DepthToSpace", ["x"], ["d2s"], blocksize=2, mode="CRD"),
        node("SpaceToDepth", ["x"], ["s2d"], blocksize=2), node("ConvTranspose", ["x", "Wt"], ["ct"], strides=[2, 2], pads=[1, 1, 1, 1], output_padding=[1, 1]),
        node("InstanceNormalization", ["x", "isc", "ibi"], ["inn"], epsilon=1e-5), node("CumSum", ["x", "ax3"], ["cs"], reverse=1),
        node("Expand", ["isc", "eshape"], ["ex"]), node("HardSwish", ["x"], ["hs"]), node("Mod", ["x", "two"], ["md"], fmod=1),
        node("Resize", ["x", "", "scales"], ["rz"], mode="nearest", coordinate_transformation_mode="asymmetric", nearest_mode="floor"),
        node("ArgMax", ["x"], ["am"], axis=1, keepdims=0), node("GatherElements", ["x", "gidx"], ["ge"], axis=3),
        node("Max", ["x", "zero", "isc4"], ["mx"]), node("Trilu", ["x"], ["tri"], upper=0),
    ]
    inits = [tensor("zero", np.zeros((), np.float32)), tensor("ax23", np.asarray([2, 3], i64)), tensor("k", np.asarray([2], i64)),
             tensor("sizes", np.asarray([1, 3], i64)), tensor("pads", np.asarray([0, 0, 1, 2, 0, 0, 2, 1], i64)), tensor("Wt", Wt.numpy()),
             tensor("isc", np.asarray([1.0, 2.0, 0.5, -1.0], np.float32)), tensor("ibi", np.asarray([0.0, 1.0, -1.0, 0.5], np.float32)),
             tensor("ax3", np.asarray(3, i64)), tensor("eshape", np.asarray([2, 3, 1], i64)), tensor("two", np.asarray(2.0, np.float32)),
             tensor("scales", np.asarray([1.0, 1.0, 2.0, 2.0], np.float32)), tensor("gidx", np.asarray(np.random.RandomState(0).randint(-6, 6, (2, 4, 6, 2)), i64)),
             tensor("isc4", np.asarray([1.0, 2.0, 0.5, -1.0], np.float32).reshape(4, 1, 1))]
    outs = ["relu_like", "l2", "lse", "tv", "ti", "s0", "s1", "pd", "d2s", "s2d", "ct", "inn", "cs", "ex", "hs", "md", "rz", "am", "ge", "mx", "tri"]
    raw = model(nodes, inits, [("x", [2, 4, 6, 6])], [(o, []) for o in outs])
    sd = OnnxFrameworkImporter(trainable=False).runImport(raw)
    r = {k: v.t for k, v in sd.output({"x": x}, *outs).items()}
    assert torch.equal(r["relu_like"], torch.where(x < 0, torch.zeros(()), x))
    assert torch.allclose(r["l2"], x.pow(2).sum(1).sqrt()) and torch.allclose(r["lse"], x.logsumexp((2, 3), keepdim=True))
    tv, ti = torch.topk(x, 2, dim=3)
    assert torch.equal(r["tv"], tv) and torch.equal(r["ti"], ti)
    assert torch.equal(r["s0"], x[:, :1]) and torch.equal(r["s1"], x[:, 1:])
    assert torch.equal(r["pd"], F.pad(x, (2, 1, 1, 2), mode="reflect"))
    assert torch.equal(r["d2s"], F.pixel_shuffle(x, 2)) and torch.equal(F.pixel_shuffle(r["s2d"].reshape(2, 2, 2, 4, 3, 3).permute(0, 3, 1, 2, 4, 5).reshape(2, 16, 3, 3), 2), x)
    assert torch.allclose(r["ct"], F.conv_transpose2d(x, Wt, stride=2, padding=1, output_padding=1), atol=1e-5)
    isc, ibi = torch.tensor([1.0, 2.0, 0.5, -1.0]), torch.tensor([0.0, 1.0, -1.0, 0.5])
    assert torch.allclose(r["inn"], F.instance_norm(x, weight=isc, bias=ibi, eps=1e-5), atol=1e-5)
    assert torch.allclose(r["cs"], x.flip(3).cumsum(3).flip(3), atol=1e-6)
    assert tuple(r["ex"].shape) == (2, 3, 4) and torch.equal(r["ex"][1, 2], isc)
    assert torch.allclose(r["hs"], F.hardswish(x), atol=1e-6) and torch.allclose(r["md"], torch.fmod(x, 2.0))
    assert torch.equal(r["rz"], x.repeat_interleave(2, 2).repeat_interleave(2, 3))
    assert torch.equal(r["am"], x.argmax(1))
    gi = torch.from_numpy(np.random.RandomState(0).randint(-6, 6, (2, 4, 6, 2)))
    assert torch.equal(r["ge"], x.gather(3, torch.where(gi < 0, gi + 6, gi)))
    assert torch.equal(r["mx"], torch.maximum(x.clamp_min(0), isc.reshape(4, 1, 1))) and torch.equal(r["tri"], torch.tril(x))


def test_lstm_and_gru_nodes_match_torch_modules():
    torch.manual_seed(0)
    T, N, I, H = 5, 3, 4, 6
    x = torch.randn(T, N, I)
    lstm = torch.nn.LSTM(I, H, bidirectional=True)
    gru = torch.nn.GRU(I, H)

    def reorder(w, order):            # torch gate blocks -> ONNX gate blocks along dim 0
        blocks = w.detach().chunk(len(order), 0)
        return torch.cat([blocks[i] for i in order], 0)
    io = [0, 3, 1, 2]                 # torch (i, f, g, o) -> ONNX (i, o, f, c)
    W = torch.stack([reorder(lstm.weight_ih_l0, io), reorder(lstm.weight_ih_l0_reverse, io)])
    R = torch.stack([reorder(lstm.weight_hh_l0, io), reorder(lstm.weight_hh_l0_reverse, io)])
    B = torch.stack([torch.cat([reorder(lstm.bias_ih_l0, io), reorder(lstm.bias_hh_l0, io)]),
                     torch.cat([reorder(lstm.bias_ih_l0_reverse, io), reorder(lstm.bias_hh_l0_reverse, io)])])
    go = [1, 0, 2]                    # torch (r, z, n) -> ONNX (z, r, h)
    Wg, Rg = reorder(gru.weight_ih_l0, go).unsqueeze(0), reorder(gru.weight_hh_l0, go).unsqueeze(0)
    Bg = torch.cat([reorder(gru.bias_ih_l0, go), reorder(gru.bias_hh_l0, go)]).unsqueeze(0)
    nodes = [node("LSTM", ["x", "W", "R", "B"], ["Y", "Yh", "Yc"], hidden_size=H, direction="bidirectional"),
             node("GRU", ["x", "Wg", "Rg", "Bg"], ["G", "Gh"], hidden_size=H, linear_before_reset=1)]
    inits = [tensor(n, t.numpy()) for n, t in (("W", W), ("R", R), ("B", B), ("Wg", Wg), ("Rg", Rg), ("Bg", Bg))]
    raw = model(nodes, inits, [("x", [T, N, I])], [("Y", []), ("Yh", []), ("Yc", []), ("G", []), ("Gh", [])])
    sd = OnnxFrameworkImporter(trainable=False).runImport(raw)
    r = {k: v.t for k, v in sd.output({"x": x}, "Y", "Yh", "Yc", "G", "Gh").items()}
    y, (h, c) = lstm(x)
    assert torch.allclose(r["Y"].permute(0, 2, 1, 3).reshape(T, N, 2 * H), y, atol=1e-5)
    assert torch.allclose(r["Yh"], h, atol=1e-5) and torch.allclose(r["Yc"], c, atol=1e-5)
    yg, hg = gru(x)
    assert torch.allclose(r["G"][:, 0], yg, atol=1e-5) and torch.allclose(r["Gh"], hg, atol=1e-5)


def test_if_and_loop_nodes_with_sub_graphs_that_read_the_outer_scope():
    then_g = graph([node("Mul", ["x", "two"], ["t_out"])], [tensor("two", np.asarray(2.0, np.float32))], [], [("t_out", [])])
    else_g = graph([node("Sub", ["x", "one"], ["e_out"])], [], [], [("e_out", [])])            # "one" and "x" come from the outer graph
    body = graph([node("Cast", ["it"], ["it_f"], to=1), node("Mul", ["x", "it_f"], ["term"]), node("Add", ["acc", "term"], ["acc_out"]),
                  node("Identity", ["cond_in"], ["cond_out"])],
                 [], [("it", []), ("cond_in", []), ("acc", [3])], [("cond_out", []), ("acc_out", [3]), ("term", [3])])
    nodes = [node("ReduceSum", ["x"], ["sx"], keepdims=0), node("Greater", ["sx", "zero"], ["pos"]),
             node("If", ["pos"], ["branch"], then_branch=then_g, else_branch=else_g),
             node("Loop", ["trip", "", "acc0"], ["acc_final", "terms"], body=body)]
    inits = [tensor("zero", np.asarray(0.0, np.float32)), tensor("one", np.asarray(1.0, np.float32)), tensor("trip", np.asarray(4, np.int64)),
             tensor("acc0", np.zeros(3, np.float32))]
    raw = model(nodes, inits, [("x", [3])], [("branch", [3]), ("acc_final", [3]), ("terms", [4, 3])])
    sd = OnnxFrameworkImporter(trainable=False).runImport(raw)
    for x in (torch.tensor([1.0, 2.0, 3.0]), torch.tensor([-1.0, -2.0, 0.5])):
        r = {k: v.t for k, v in sd.output({"x": x}, "branch", "acc_final", "terms").items()}
        assert torch.equal(r["branch"], x * 2 if float(x.sum()) > 0 else x - 1)
        assert torch.equal(r["acc_final"], x * (0 + 1 + 2 + 3)) and tuple(r["terms"].shape) == (4, 3) and torch.equal(r["terms"][2], x * 2)


def test_remaining_standard_operators_by_their_definitions():
    """Compress, Det, Shrink, GroupNormalization, Quantize / DequantizeLinear, ReverseSequence, Unique, RNN, NonMaxSuppression and
    RoiAlign: each rule against the operator's definition written out with plain torch."""
    from deeplearning4j_b200.importers.onnx_import import _onnx_ops
    T = {k: v[0] for k, v in _onnx_ops().items()}
    g = torch.Generator().manual_seed(5)
    x = torch.randn(3, 4, generator=g)
    assert torch.equal(T["Compress"](x, torch.tensor([0, 1, 1]), axis=0), x[1:3])
    assert torch.equal(T["Compress"](x, torch.tensor([0, 1, 0, 0, 1])), x.reshape(-1)[[1, 4]])
    m = torch.randn(2, 3, 3, generator=g)
    torch.testing.assert_close(T["Det"](m), torch.stack([torch.det(m[0]), torch.det(m[1])]))
    s = T["Shrink"](torch.tensor([-2.0, -0.3, 0.0, 0.4, 3.0]), bias=1.0, lambd=0.5)
    assert s.tolist() == [-1.0, 0.0, 0.0, 0.0, 2.0]
    xg = torch.randn(2, 6, 5, generator=g)
    sc, b = torch.rand(6, generator=g) + 0.5, torch.randn(6, generator=g)
    torch.testing.assert_close(T["GroupNormalization"](xg, sc, b, num_groups=3, epsilon=1e-5), F.group_norm(xg, 3, sc, b, 1e-5))
    q = T["QuantizeLinear"](torch.tensor([[0.0, 1.0, 300.0], [-1.0, 2.49, 2.51]]), torch.tensor(2.0), torch.tensor(3, dtype=torch.uint8))
    assert q.dtype == torch.uint8 and q.tolist() == [[3, 3, 153], [3, 4, 4]]        # x / 2 rounded half to even (0.5 -> 0, -0.5 -> -0), plus 3
    d = T["DequantizeLinear"](torch.tensor([[0, 10], [20, 30]], dtype=torch.int8), torch.tensor([0.5, 2.0]), torch.tensor([0, 10], dtype=torch.int8), axis=1)
    assert d.tolist() == [[0.0, 0.0], [10.0, 40.0]]
    seq = torch.arange(12.0).reshape(4, 3)                                         # [time, batch]
    r = T["ReverseSequence"](seq, torch.tensor([4, 2, 1]), batch_axis=1, time_axis=0)
    assert r[:, 0].tolist() == [9.0, 6.0, 3.0, 0.0] and r[:, 1].tolist() == [4.0, 1.0, 7.0, 10.0] and r[:, 2].tolist() == [2.0, 5.0, 8.0, 11.0]
    y, first, inv, cnt = T["Unique"](torch.tensor([2.0, 1.0, 1.0, 3.0, 4.0, 3.0]), sorted=1)
    assert y.tolist() == [1.0, 2.0, 3.0, 4.0] and first.tolist() == [1, 0, 3, 4] and inv.tolist() == [1, 0, 0, 2, 3, 2] and cnt.tolist() == [2, 1, 2, 1]
    y, first, inv, cnt = T["Unique"](torch.tensor([2.0, 1.0, 1.0, 3.0, 4.0, 3.0]), sorted=0)
    assert y.tolist() == [2.0, 1.0, 3.0, 4.0] and first.tolist() == [0, 1, 3, 4] and inv.tolist() == [0, 1, 1, 2, 3, 2] and cnt.tolist() == [1, 2, 2, 1]
    # RNN against torch.nn.RNN
    rnn = torch.nn.RNN(3, 4, nonlinearity="tanh")
    xs = torch.randn(5, 2, 3, generator=g)
    ref_y, ref_h = rnn(xs)
    W, R = rnn.weight_ih_l0.detach()[None], rnn.weight_hh_l0.detach()[None]
    B = torch.cat([rnn.bias_ih_l0.detach(), rnn.bias_hh_l0.detach()])[None]
    Y, Yh = T["RNN"](xs, W, R, B, hidden_size=4)
    torch.testing.assert_close(Y[:, 0], ref_y.detach(), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(Yh, ref_h.detach(), rtol=1e-5, atol=1e-6)
    # NonMaxSuppression: the second box overlaps the first (IoU 0.68) and is suppressed, the third is far away
    boxes = torch.tensor([[[0.0, 0.0, 1.0, 1.0], [0.0, 0.1, 1.0, 1.1], [0.0, 2.0, 1.0, 3.0]]])
    scores = torch.tensor([[[0.9, 0.8, 0.7]]])
    sel = T["NonMaxSuppression"](boxes, scores, torch.tensor([3]), torch.tensor([0.5]), torch.tensor([0.0]))
    assert sel.tolist() == [[0, 0, 0], [0, 0, 2]]
    # RoiAlign: a roi covering one whole 4x4 image pooled to 2x2 with one sample per bin reads the bin centres
    img = torch.arange(16.0).reshape(1, 1, 4, 4)
    ra = T["RoiAlign"](img, torch.tensor([[0.0, 0.0, 4.0, 4.0]]), torch.tensor([0]), output_height=2, output_width=2, sampling_ratio=1,
                       coordinate_transformation_mode="output_half_pixel")
    # bin centres (1, 1), (1, 3), (3, 1), (3, 3) in input coordinates fall exactly on pixels
    ref = torch.tensor([[img[0, 0, 1, 1], img[0, 0, 1, 3]], [img[0, 0, 3, 1], img[0, 0, 3, 3]]])
    torch.testing.assert_close(ra[0, 0], ref)


def test_second_operator_table_by_definitions():
    """Integer / quantised linear algebra, windows and spectral ops, unpooling, losses: each against the operator's definition in the
    ONNX specification written out in plain torch / numpy."""
    import math
    import torch.nn.functional as F
    from deeplearning4j_b200.importers.onnx_import import _onnx_ops
    T = {k: v[0] for k, v in _onnx_ops().items()}
    g = torch.Generator().manual_seed(3)

    w = T["HannWindow"](torch.tensor(8))
    assert torch.allclose(w, torch.hann_window(8, periodic=True)) and torch.allclose(T["HannWindow"](torch.tensor(8), periodic=0), torch.hann_window(8, periodic=False))
    assert torch.allclose(T["HammingWindow"](torch.tensor(6), periodic=0), torch.tensor([25 / 46 - 21 / 46 * math.cos(2 * math.pi * k / 5) for k in range(6)]))
    assert torch.allclose(T["BlackmanWindow"](torch.tensor(7)), torch.blackman_window(7, periodic=True), atol=1e-6)
    assert T["BitwiseNot"](torch.tensor([0, 5], dtype=torch.uint8)).tolist() == [255, 250] and T["CastLike"](torch.tensor([1.7]), torch.tensor([1])).dtype == torch.int64

    x = torch.randint(0, 255, (1, 2, 5, 5), generator=g, dtype=torch.uint8)
    wt = torch.randint(-100, 100, (3, 2, 3, 3), generator=g, dtype=torch.int8)
    ref = F.conv2d(x.double() - 7, wt.double(), padding=1)
    assert torch.equal(T["ConvInteger"](x, wt, torch.tensor(7, dtype=torch.uint8), pads=[1, 1, 1, 1]), ref.to(torch.int32))
    a = torch.randint(0, 255, (4, 6), generator=g, dtype=torch.uint8)
    b = torch.randint(-128, 127, (6, 3), generator=g, dtype=torch.int8)
    assert torch.equal(T["MatMulInteger"](a, b, torch.tensor(12, dtype=torch.uint8)), ((a.long() - 12) @ b.long()).to(torch.int32))
    q = T["QLinearMatMul"](a, torch.tensor(0.1), torch.tensor(12, dtype=torch.uint8), b, torch.tensor(0.05), torch.tensor(0, dtype=torch.int8),
                           torch.tensor(2.0), torch.tensor(100, dtype=torch.uint8))
    assert torch.equal(q, torch.clamp(torch.round(((a.double() - 12) @ b.double()) * 0.1 * 0.05 / 2.0) + 100, 0, 255).to(torch.uint8))
    qc = T["QLinearConv"](x, torch.tensor(0.02), torch.tensor(7, dtype=torch.uint8), wt, torch.tensor(0.01), torch.tensor(0, dtype=torch.int8),
                          torch.tensor(0.5), torch.tensor(3, dtype=torch.uint8), torch.tensor([5, -5, 0], dtype=torch.int32), pads=[1, 1, 1, 1])
    refq = torch.clamp(torch.round((ref + torch.tensor([5.0, -5, 0]).reshape(1, 3, 1, 1)) * 0.02 * 0.01 / 0.5) + 3, 0, 255).to(torch.uint8)
    assert torch.equal(qc, refq)
    y, sc, zp = T["DynamicQuantizeLinear"](torch.tensor([0.0, 2.0, -3.0, -2.5, 1.34, 0.5]))
    assert float(sc) == pytest.approx(5.0 / 255) and int(zp) == 153 and y.tolist() == [153, 255, 0, 26, 221, 179]      # the specification's own example

    img = torch.randn(2, 3, 6, 6, generator=g)
    lp = T["LpPool"](img, kernel_shape=[2, 2], strides=[2, 2], p=3)
    assert torch.allclose(lp, (F.avg_pool2d(img.abs() ** 3, 2) * 4) ** (1 / 3), atol=1e-5)
    pooled, idx = F.max_pool2d(img, 2, return_indices=True)
    flat = idx + (torch.arange(2 * 3).reshape(2, 3, 1, 1) * 36)                         # ONNX indices address the whole tensor
    un = T["MaxUnpool"](pooled, flat, kernel_shape=[2, 2], strides=[2, 2])
    assert torch.equal(un, F.max_unpool2d(pooled, idx, 2))
    rp = T["MaxRoiPool"](img, torch.tensor([[1.0, 0, 0, 3, 3], [0.0, 2, 2, 5, 5]]), pooled_shape=[2, 2], spatial_scale=1.0)
    assert torch.equal(rp[0], F.max_pool2d(img[1, :, 0:4, 0:4], 2)) and torch.equal(rp[1], F.max_pool2d(img[0, :, 2:6, 2:6], 2))
    grid = torch.rand(2, 4, 4, 2, generator=g) * 2 - 1
    assert torch.allclose(T["GridSample"](img, grid, mode=b"linear", align_corners=1), F.grid_sample(img, grid, align_corners=True))
    cols = F.unfold(img, (2, 2), stride=2)
    assert torch.equal(T["Col2Im"](cols, torch.tensor([6, 6]), torch.tensor([2, 2]), strides=[2, 2]), img)
    cc = T["CenterCropPad"](img, torch.tensor([4, 8]), axes=[2, 3])
    assert cc.shape == (2, 3, 4, 8) and torch.equal(cc[:, :, :, 1:7], img[:, :, 1:5, :]) and cc[:, :, :, 0].abs().sum() == 0

    logits = torch.randn(5, 4, generator=g)
    labels = torch.tensor([0, 3, 1, 1, 2])
    loss, logp = T["SoftmaxCrossEntropyLoss"](logits, labels, reduction=b"mean")
    assert torch.allclose(loss, F.cross_entropy(logits, labels)) and torch.allclose(logp, logits.log_softmax(1))
    wts = torch.tensor([1.0, 2.0, 0.5, 1.5])
    assert torch.allclose(T["NegativeLogLikelihoodLoss"](logits.log_softmax(1), labels, wts, reduction=b"sum", ignore_index=1),
                          F.nll_loss(logits.log_softmax(1), labels, wts, ignore_index=1, reduction="sum"))

    sig = torch.randn(2, 16, 1, generator=g)
    assert torch.allclose(T["DFT"](sig, axis=1), torch.view_as_real(torch.fft.fft(sig[..., 0], dim=1)), atol=1e-5)
    assert torch.allclose(T["DFT"](sig, axis=1, onesided=1), torch.view_as_real(torch.fft.rfft(sig[..., 0], dim=1)), atol=1e-5)
    spec = T["DFT"](sig, axis=1)
    assert torch.allclose(T["DFT"](spec, axis=1, inverse=1)[..., 0], sig[..., 0], atol=1e-5)
    st = T["STFT"](sig, torch.tensor(4), torch.hann_window(8), torch.tensor(8))
    ref = torch.stft(sig[..., 0], 8, 4, window=torch.hann_window(8), center=False, return_complex=True).transpose(1, 2)
    assert torch.allclose(st, torch.view_as_real(ref), atol=1e-5)
    mw = T["MelWeightMatrix"](torch.tensor(8), torch.tensor(16), torch.tensor(8192), torch.tensor(0.0), torch.tensor(4096.0))
    assert mw.shape == (9, 8) and float(mw.max()) == 1.0 and float(mw.min()) == 0.0 and bool((mw.sum(0) > 0).all())

    r1 = T["RandomNormal"](shape=[1000], mean=2.0, scale=0.5, seed=1.0)
    assert r1.shape == (1000,) and abs(float(r1.mean()) - 2.0) < 0.1 and torch.equal(r1, T["RandomNormal"](shape=[1000], mean=2.0, scale=0.5, seed=1.0))
    r2 = T["RandomUniformLike"](torch.zeros(3, 4, dtype=torch.float64), low=2.0, high=3.0)
    assert r2.dtype == torch.float64 and float(r2.min()) >= 2.0 and float(r2.max()) < 3.0
    assert set(T["Bernoulli"](torch.full((50,), 0.5), seed=2.0).tolist()) <= {0.0, 1.0}
    assert T["Multinomial"](torch.tensor([[0.0, 50.0, 0.0]]), sample_size=5).tolist() == [[1] * 5]
