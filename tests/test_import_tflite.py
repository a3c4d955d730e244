"""TFLite flatbuffer import.  The models are written with the same schema tables the importer reads (no TFLite runtime exists
here), and every operator is checked against the TensorFlow semantics restated with plain torch calls."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from deeplearning4j_b200.importers.tflite_import import (BUILTIN_CODES, OPTION_IDS, TENSOR_TYPE_IDS, TFL_SCHEMA, importTFLite, supportedOps)
from deeplearning4j_b200.samediff.serde.flatbuffers import decode, encode


class ModelBuilder:
    """Collects tensors / operators and writes a ``TFL3`` file."""

    def __init__(self):
        self.tensors, self.buffers, self.ops, self.codes = [], [{}], [], []

    def tensor(self, name, shape, dtype=torch.float32, data=None, quantization=None):
        t = {"shape": list(shape), "type": TENSOR_TYPE_IDS[dtype], "name": name, "buffer": 0}
        if data is not None:
            arr = data.detach().to(dtype).contiguous()
            self.buffers.append({"data": arr.numpy().tobytes()})
            t["buffer"] = len(self.buffers) - 1
        if quantization is not None:
            t["quantization"] = quantization
        self.tensors.append(t)
        return len(self.tensors) - 1

    def op(self, kind, inputs, outputs, options=None, **opts):
        code = BUILTIN_CODES[kind]
        if code not in self.codes:
            self.codes.append(code)
        o = {"opcode_index": self.codes.index(code), "inputs": list(inputs), "outputs": list(outputs)}
        if options is not None:
            o["builtin_options_type"] = OPTION_IDS[options]
            o["builtin_options"] = opts
        self.ops.append(o)

    def build(self, inputs, outputs):
        model = {"version": 3, "description": "test",
                 "operator_codes": [{"deprecated_builtin_code": min(c, 127), "builtin_code": c} for c in self.codes],
                 "subgraphs": [{"tensors": self.tensors, "inputs": list(inputs), "outputs": list(outputs), "operators": self.ops, "name": "main"}],
                 "buffers": self.buffers}
        return encode("Model", model, schema=TFL_SCHEMA, identifier=b"TFL3")


def _run(data, feeds, outs=None):
    sd = importTFLite(data)
    outs = outs or sd.metadata["tflite.outputs"].split(",")
    res = sd.output(feeds, *outs)
    return [res[o].t if hasattr(res[o], "t") else res[o] for o in outs]


def _tf_same(x, k, s):
    out = -(-x // s)
    total = max((out - 1) * s + k - x, 0)
    return total // 2, total - total // 2


def test_flatbuffer_round_trip_with_union_and_defaults():
    b = ModelBuilder()
    x = b.tensor("x", [1, 5, 5, 2])
    w = b.tensor("w", [3, 3, 3, 2], data=torch.ones(3, 3, 3, 2))
    y = b.tensor("y", [1, 3, 3, 3])
    b.op("CONV_2D", [x, w, -1], [y], "Conv2DOptions", padding=0, stride_w=2, stride_h=2, fused_activation_function=1)
    data = b.build([x], [y])
    assert data[4:8] == b"TFL3"
    m = decode("Model", data, schema=TFL_SCHEMA)
    o = m["subgraphs"][0]["operators"][0]
    assert o["builtin_options"]["stride_w"] == 2 and o["builtin_options"]["dilation_w_factor"] == 1      # schema default
    assert list(o["inputs"]) == [0, 1, -1]
    assert m["operator_codes"][0]["version"] == 1


def test_small_cnn_matches_torch():
    g = torch.Generator().manual_seed(0)
    w1, b1 = torch.randn(8, 3, 3, 3, generator=g) * 0.3, torch.randn(8, generator=g) * 0.1
    wd = torch.randn(1, 3, 3, 8, generator=g) * 0.3
    wf, bf = torch.randn(10, 8, generator=g) * 0.3, torch.randn(10, generator=g) * 0.1
    b = ModelBuilder()
    x = b.tensor("input", [2, 9, 9, 3])
    t_w1, t_b1 = b.tensor("w1", w1.shape, data=w1), b.tensor("b1", b1.shape, data=b1)
    c1 = b.tensor("c1", [2, 5, 5, 8])
    b.op("CONV_2D", [x, t_w1, t_b1], [c1], "Conv2DOptions", padding=0, stride_w=2, stride_h=2, fused_activation_function=3)
    t_wd = b.tensor("wd", wd.shape, data=wd)
    d1 = b.tensor("d1", [2, 5, 5, 8])
    b.op("DEPTHWISE_CONV_2D", [c1, t_wd, -1], [d1], "DepthwiseConv2DOptions", padding=0, stride_w=1, stride_h=1, depth_multiplier=1)
    p1 = b.tensor("p1", [2, 3, 3, 8])
    b.op("AVERAGE_POOL_2D", [d1], [p1], "Pool2DOptions", padding=0, stride_w=2, stride_h=2, filter_width=2, filter_height=2)
    p2 = b.tensor("p2", [2, 2, 2, 8])
    b.op("MAX_POOL_2D", [p1], [p2], "Pool2DOptions", padding=1, stride_w=1, stride_h=1, filter_width=2, filter_height=2)
    ax = b.tensor("axes", [2], torch.int32, data=torch.tensor([1, 2]))
    m = b.tensor("gap", [2, 8])
    b.op("MEAN", [p2, ax], [m], "ReducerOptions", keep_dims=False)
    t_wf, t_bf = b.tensor("wf", wf.shape, data=wf), b.tensor("bf", bf.shape, data=bf)
    fc = b.tensor("logits", [2, 10])
    b.op("FULLY_CONNECTED", [m, t_wf, t_bf], [fc], "FullyConnectedOptions", fused_activation_function=0)
    sm = b.tensor("probabilities", [2, 10])
    b.op("SOFTMAX", [fc], [sm], "SoftmaxOptions", beta=1.0)
    data = b.build([x], [sm])

    xin = torch.randn(2, 9, 9, 3, generator=g)
    got, = _run(data, {"input": xin})
    xn = xin.permute(0, 3, 1, 2)
    (t, bt), (l, r) = _tf_same(9, 3, 2), _tf_same(9, 3, 2)
    y = F.conv2d(F.pad(xn, (l, r, t, bt)), w1.permute(0, 3, 1, 2), b1, 2).clamp(0, 6)
    y = F.conv2d(F.pad(y, (1, 1, 1, 1)), wd.permute(3, 0, 1, 2), None, 1, groups=8)
    pad = F.pad(y, (0, 1, 0, 1))                                                       # SAME 2x2 stride 2 on 5x5: one cell at the end
    cnt = F.avg_pool2d(F.pad(torch.ones(1, 1, 5, 5), (0, 1, 0, 1)), 2, 2)
    y = F.avg_pool2d(pad, 2, 2) / cnt
    y = F.max_pool2d(y, 2, 1)
    y = y.mean((2, 3)) @ wf.t() + bf
    torch.testing.assert_close(got, torch.softmax(y, -1), rtol=1e-4, atol=1e-5)


def test_shape_and_elementwise_operators():
    g = torch.Generator().manual_seed(1)
    b = ModelBuilder()
    x = b.tensor("x", [2, 4, 6])
    y = b.tensor("y", [2, 4, 6])
    s = b.tensor("sum", [2, 4, 6]); b.op("ADD", [x, y], [s], "AddOptions", fused_activation_function=1)
    shp = b.tensor("shape", [2], torch.int32, data=torch.tensor([8, 6]))
    r = b.tensor("r", [8, 6]); b.op("RESHAPE", [s, shp], [r], "ReshapeOptions", new_shape=[8, 6])
    perm = b.tensor("perm", [2], torch.int32, data=torch.tensor([1, 0]))
    tr = b.tensor("tr", [6, 8]); b.op("TRANSPOSE", [r, perm], [tr])
    bg, en, st = (b.tensor(n, [2], torch.int32, data=torch.tensor(v)) for n, v in (("bg", [1, 0]), ("en", [5, 0]), ("st", [2, 1])))
    ss = b.tensor("ss", [2, 8]); b.op("STRIDED_SLICE", [tr, bg, en, st], [ss], "StridedSliceOptions", end_mask=2)
    cat = b.tensor("cat", [4, 8]); b.op("CONCATENATION", [ss, ss], [cat], "ConcatenationOptions", axis=0)
    pads = b.tensor("pads", [2, 2], torch.int32, data=torch.tensor([[1, 0], [0, 2]]))
    pd = b.tensor("pd", [5, 10]); b.op("PAD", [cat, pads], [pd])
    gl = b.tensor("gelu", [5, 10]); b.op("GELU", [pd], [gl], "GeluOptions", approximate=True)
    ax = b.tensor("ax", [], torch.int32, data=torch.tensor(1))
    am = b.tensor("am", [5], torch.int64); b.op("ARG_MAX", [gl, ax], [am], "ArgMaxOptions", output_type=4)
    o1, o2 = b.tensor("u0", [10]), b.tensor("u1", [10])
    rows = b.tensor("rows", [2, 10])
    b0, sz = b.tensor("b0", [2], torch.int32, data=torch.tensor([1, 0])), b.tensor("sz", [2], torch.int32, data=torch.tensor([2, -1]))
    b.op("SLICE", [gl, b0, sz], [rows])
    b.op("UNPACK", [rows], [o1, o2], "UnpackOptions", num=2, axis=0)
    lk = b.tensor("leaky", [10]); b.op("LEAKY_RELU", [o2], [lk], "LeakyReluOptions", alpha=0.2)
    data = b.build([x, y], [am, o1, lk])
    xv, yv = torch.randn(2, 4, 6, generator=g), torch.randn(2, 4, 6, generator=g)
    am_, o1_, lk_ = _run(data, {"x": xv, "y": yv})
    ref = torch.relu(xv + yv).reshape(8, 6).t()[1:5:2, :]
    ref = F.pad(torch.cat([ref, ref], 0), (0, 2, 1, 0))
    ref = F.gelu(ref, approximate="tanh")
    assert am_.dtype == torch.int64 and torch.equal(am_, ref.argmax(1))
    torch.testing.assert_close(o1_, ref[1])
    torch.testing.assert_close(lk_, F.leaky_relu(ref[2], 0.2))


def test_quantised_and_half_weights_are_dequantised():
    g = torch.Generator().manual_seed(2)
    q = torch.randint(-127, 128, (4, 6), generator=g, dtype=torch.int8)
    scale = torch.tensor([0.01, 0.02, 0.03, 0.04])
    b = ModelBuilder()
    x = b.tensor("x", [3, 6])
    w = b.tensor("w", [4, 6], torch.int8, data=q, quantization={"scale": scale.tolist(), "zero_point": [0, 0, 0, 0], "quantized_dimension": 0})
    hb = torch.randn(4, generator=g).half()
    bias = b.tensor("bias", [4], torch.float16, data=hb)
    y = b.tensor("y", [3, 4]); b.op("FULLY_CONNECTED", [x, w, bias], [y], "FullyConnectedOptions", fused_activation_function=4)
    data = b.build([x], [y])
    xv = torch.randn(3, 6, generator=g)
    got, = _run(data, {"x": xv})
    torch.testing.assert_close(got, torch.tanh(xv @ (q.float() * scale[:, None]).t() + hb.float()), rtol=1e-5, atol=1e-6)


def test_resize_transpose_conv_and_batch_matmul():
    g = torch.Generator().manual_seed(3)
    b = ModelBuilder()
    x = b.tensor("x", [1, 4, 4, 2])
    size = b.tensor("size", [2], torch.int32, data=torch.tensor([8, 8]))
    up = b.tensor("up", [1, 8, 8, 2]); b.op("RESIZE_BILINEAR", [x, size], [up], "ResizeBilinearOptions", half_pixel_centers=True)
    nn_ = b.tensor("nn", [1, 8, 8, 2]); b.op("RESIZE_NEAREST_NEIGHBOR", [x, size], [nn_], "ResizeNearestNeighborOptions")
    wt = torch.randn(3, 2, 2, 2, generator=g)
    t_w = b.tensor("wt", wt.shape, data=wt)
    osh = b.tensor("osh", [4], torch.int32, data=torch.tensor([1, 8, 8, 3]))
    tc = b.tensor("tc", [1, 8, 8, 3]); b.op("TRANSPOSE_CONV", [osh, t_w, x], [tc], "TransposeConvOptions", padding=1, stride_w=2, stride_h=2)
    a, c = b.tensor("a", [2, 3, 5]), b.tensor("c", [2, 4, 5])
    mm = b.tensor("mm", [2, 3, 4]); b.op("BATCH_MATMUL", [a, c], [mm], "BatchMatMulOptions", adj_y=True)
    data = b.build([x, a, c], [up, nn_, tc, mm])
    xv, av, cv = torch.randn(1, 4, 4, 2, generator=g), torch.randn(2, 3, 5, generator=g), torch.randn(2, 4, 5, generator=g)
    up_, nn__, tc_, mm_ = _run(data, {"x": xv, "a": av, "c": cv})
    xn = xv.permute(0, 3, 1, 2)
    torch.testing.assert_close(up_, F.interpolate(xn, size=(8, 8), mode="bilinear", align_corners=False).permute(0, 2, 3, 1), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(nn__, F.interpolate(xn, size=(8, 8), mode="nearest").permute(0, 2, 3, 1))
    torch.testing.assert_close(tc_, F.conv_transpose2d(xn, wt.permute(3, 0, 1, 2), None, 2).permute(0, 2, 3, 1), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(mm_, av @ cv.transpose(1, 2))


def test_runner_and_errors(tmp_path):
    from deeplearning4j_b200.runtimes import TensorFlowLiteRunner
    b = ModelBuilder()
    x = b.tensor("x", [2, 3])
    y = b.tensor("y", [2, 3]); b.op("LOGISTIC", [x], [y])
    p = tmp_path / "m.tflite"
    p.write_bytes(b.build([x], [y]))
    with TensorFlowLiteRunner.builder().modelUri(str(p)).build() as r:
        assert r.getInputs() == ["x"] and r.getOutputs() == ["y"]
        out = r.exec({"x": torch.zeros(2, 3)})
        assert torch.allclose(out["y"].t, torch.full((2, 3), 0.5))
    bad = ModelBuilder()
    bad.codes.append(27)                                # SVDF: no rule
    bad.tensors.append({"shape": [1], "type": 0, "name": "x", "buffer": 0})
    bad.ops.append({"opcode_index": 0, "inputs": [0], "outputs": [0]})
    with pytest.raises(NotImplementedError, match="builtin#27"):
        importTFLite(bad.build([0], [0]))
    assert len(supportedOps()) >= 90


def test_further_builtin_operators_by_definitions():
    """Builtin operators added after the first table (space / batch, segment, scatter, top-k, ...), each against its definition."""
    import torch
    from deeplearning4j_b200.importers.tflite_import import _tflite_ops, supportedOps
    T = {k: v[0] for k, v in _tflite_ops().items()}
    assert len(supportedOps()) >= 114
    x = torch.arange(1 * 4 * 6 * 2, dtype=torch.float32).reshape(1, 4, 6, 2)
    zero = torch.zeros(2, 2, dtype=torch.int64)
    y = T["SPACE_TO_BATCH_ND"](x, torch.tensor([2, 2]), zero)
    assert torch.equal(y[3], x[0, 1::2, 1::2]) and torch.equal(T["BATCH_TO_SPACE_ND"](y, torch.tensor([2, 2]), zero), x)
    ref = torch.nn.functional.avg_pool2d((x * x).permute(0, 3, 1, 2), 2).sqrt().permute(0, 2, 3, 1)
    assert torch.allclose(T["L2_POOL_2D"](x, padding=1, stride_w=2, stride_h=2, filter_width=2, filter_height=2), ref)
    v, i = T["TOPK_V2"](torch.tensor([[1.0, 5, 3]]), torch.tensor(2))
    assert v.tolist() == [[5, 3]] and i.tolist() == [[1, 2]]
    assert T["SPARSE_TO_DENSE"](torch.tensor([[0, 1], [1, 0]]), torch.tensor([2, 2]), torch.tensor([5.0, 6]), torch.tensor(-1.0)).tolist() == [[-1, 5], [6, -1]]
    assert T["REDUCE_ANY"](torch.tensor([[True, False], [False, False]]), torch.tensor([1])).tolist() == [True, False]
    assert T["REDUCE_ALL"](torch.tensor([[True, True], [True, False]]), torch.tensor([1])).tolist() == [True, False]
    assert T["WHERE"](torch.tensor([True, False, True])).tolist() == [[0], [2]]
    assert T["MATRIX_DIAG"](torch.tensor([1.0, 2])).tolist() == [[1, 0], [0, 2]] and T["MATRIX_SET_DIAG"](torch.zeros(2, 2), torch.tensor([1.0, 2])).tolist() == [[1, 0], [0, 2]]
    assert T["SCATTER_ND"](torch.tensor([[1], [1]]), torch.tensor([2.0, 3]), torch.tensor([3])).tolist() == [0, 5, 0]
    d = torch.tensor([[1.0, 2], [3, 4], [5, 6]])
    assert T["SEGMENT_SUM"](d, torch.tensor([0, 0, 1])).tolist() == [[4, 6], [5, 6]]
    assert T["UNSORTED_SEGMENT_SUM"](d, torch.tensor([1, -1, 1]), torch.tensor(2)).tolist() == [[0, 0], [6, 8]]
    assert T["UNSORTED_SEGMENT_MAX"](d, torch.tensor([1, 0, 1]), torch.tensor(2)).tolist() == [[3, 4], [5, 6]]
    assert T["UNSORTED_SEGMENT_MIN"](d, torch.tensor([1, 0, 1]), torch.tensor(2)).tolist() == [[3, 4], [1, 2]]
    assert T["UNSORTED_SEGMENT_PROD"](d, torch.tensor([1, 0, 1]), torch.tensor(2)).tolist() == [[3, 4], [5, 12]]
    assert T["BROADCAST_ARGS"](torch.tensor([3, 1]), torch.tensor([1, 4])).tolist() == [3, 4] and T["BROADCAST_TO"](torch.tensor([1.0, 2]), torch.tensor([2, 2])).tolist() == [[1, 2], [1, 2]]
    assert T["RELU_0_TO_1"](torch.tensor([-1.0, 0.5, 2])).tolist() == [0, 0.5, 1] and T["SIGN"](torch.tensor([-2.0, 0, 3])).tolist() == [-1, 0, 1]
    assert torch.allclose(T["ATAN2"](torch.tensor([1.0]), torch.tensor([-1.0])), torch.tensor([3 * 3.141592653589793 / 4]))
