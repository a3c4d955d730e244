"""TensorFlow GraphDef and Keras imports checked against torch computations of the same networks."""
import json
import struct

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from deeplearning4j_b200.importers import KerasModelImport, TensorflowFrameworkImporter, UnsupportedKerasConfigurationException
from deeplearning4j_b200.importers import protowire as pw


# ----------------------------------------------------------------------------- TF GraphDef encoding helpers
def tf_tensor(arr):
    arr = np.ascontiguousarray(arr)
    dt = {np.dtype("float32"): 1, np.dtype("int32"): 3}[arr.dtype]
    shape = b"".join(pw.field_bytes(2, pw.field_varint(1, d)) for d in arr.shape)
    return pw.field_varint(1, dt) + pw.field_bytes(2, shape) + pw.field_bytes(4, arr.tobytes())


def tf_attr(v):
    if isinstance(v, np.ndarray):
        return pw.field_bytes(8, tf_tensor(v))
    if isinstance(v, bool):
        return pw.field_varint(5, int(v))
    if isinstance(v, str):
        return pw.field_bytes(2, v.encode())
    if isinstance(v, int):
        return pw.field_varint(3, v)
    if isinstance(v, float):
        return pw.field_float(4, v)
    if isinstance(v, list):
        return pw.field_bytes(1, pw.field_packed_varints(3, v))
    if isinstance(v, tuple) and v[0] == "dtype":
        return pw.field_varint(6, v[1])
    if isinstance(v, tuple) and v[0] == "shape":
        return pw.field_bytes(7, b"".join(pw.field_bytes(2, pw.field_varint(1, d)) for d in v[1]))
    raise TypeError(v)


def tf_node(name, op, inputs=(), **attrs):
    b = pw.field_string(1, name) + pw.field_string(2, op) + b"".join(pw.field_string(3, i) for i in inputs)
    for k, v in attrs.items():
        b += pw.field_bytes(5, pw.field_string(1, k) + pw.field_bytes(2, tf_attr(v)))
    return pw.field_bytes(1, b)


def test_tensorflow_graphdef_cnn():
    g = torch.Generator().manual_seed(0)
    K = torch.randn(3, 3, 2, 4, generator=g) * 0.3                     # HWIO
    b = torch.randn(4, generator=g) * 0.1
    W = torch.randn(4 * 4 * 4, 3, generator=g) * 0.1
    graph = b"".join([
        tf_node("x", "Placeholder", dtype=("dtype", 1), shape=("shape", [1, 8, 8, 2])),
        tf_node("K", "Const", value=K.numpy()), tf_node("b", "Const", value=b.numpy()), tf_node("W", "Const", value=W.numpy()),
        tf_node("shape", "Const", value=np.asarray([-1, 64], dtype=np.int32)),
        tf_node("conv", "Conv2D", ["x", "K"], strides=[1, 1, 1, 1], padding="SAME", data_format="NHWC"),
        tf_node("bias", "BiasAdd", ["conv", "b"]), tf_node("relu", "Relu", ["bias"]),
        tf_node("pool", "MaxPool", ["relu"], ksize=[1, 2, 2, 1], strides=[1, 2, 2, 1], padding="VALID"),
        tf_node("flat", "Reshape", ["pool", "shape"]), tf_node("logits", "MatMul", ["flat", "W"], transpose_b=False),
        tf_node("prob", "Softmax", ["logits", "^relu"])])
    imp = TensorflowFrameworkImporter()
    sd = imp.runImport(graph)
    assert imp.outputs == ["prob"]
    x = torch.randn(2, 8, 8, 2, generator=g)
    got = sd.output({"x": x}, "prob")["prob"].t
    h = F.relu(F.conv2d(x.permute(0, 3, 1, 2), K.permute(3, 2, 0, 1), b, padding=1))
    h = F.max_pool2d(h, 2).permute(0, 2, 3, 1).reshape(2, -1)
    assert torch.allclose(got, F.softmax(h @ W, -1), atol=1e-5)
    with pytest.raises(NotImplementedError, match="TensorArrayV3"):
        TensorflowFrameworkImporter().runImport(tf_node("t", "TensorArrayV3"))


# ----------------------------------------------------------------------------- Keras
def _seq_json(layers, loss=None):
    d = {"class_name": "Sequential", "config": {"name": "seq", "layers": layers}}
    if loss:
        d["training_config"] = {"loss": loss}
    return json.dumps(d)


def test_keras_sequential_cnn_matches_manual_forward():
    g = torch.Generator().manual_seed(1)
    K = torch.randn(3, 3, 2, 4, generator=g) * 0.3
    kb = torch.randn(4, generator=g) * 0.1
    gamma, beta, mean, var = torch.rand(4, generator=g) + 0.5, torch.randn(4, generator=g) * 0.1, torch.randn(4, generator=g) * 0.1, torch.rand(4, generator=g) + 0.5
    W = torch.randn(3 * 3 * 4, 5, generator=g) * 0.2
    wb = torch.randn(5, generator=g) * 0.1
    layers = [{"class_name": "Conv2D", "config": {"name": "c1", "filters": 4, "kernel_size": [3, 3], "strides": [1, 1], "padding": "valid", "activation": "relu",
                                                  "use_bias": True, "batch_input_shape": [None, 8, 8, 2]}},
              {"class_name": "BatchNormalization", "config": {"name": "bn", "epsilon": 1e-3, "momentum": 0.99}},
              {"class_name": "MaxPooling2D", "config": {"name": "p1", "pool_size": [2, 2], "strides": [2, 2], "padding": "valid"}},
              {"class_name": "Dropout", "config": {"name": "do", "rate": 0.25}},
              {"class_name": "Flatten", "config": {"name": "fl"}},
              {"class_name": "Dense", "config": {"name": "d1", "units": 5, "activation": "softmax", "use_bias": True}}]
    weights = {"c1": [K.numpy(), kb.numpy()], "bn": [gamma.numpy(), beta.numpy(), mean.numpy(), var.numpy()], "d1": [W.numpy(), wb.numpy()]}
    net = KerasModelImport.importKerasSequentialModelAndWeights(_seq_json(layers, "categorical_crossentropy"), weights)
    assert [type(l).__name__ for l in net.conf.layers()] == ["ConvolutionLayer", "BatchNormalization", "SubsamplingLayer", "DropoutLayer", "OutputLayer"]
    x_nhwc = torch.randn(3, 8, 8, 2, generator=g)
    got = net.output(x_nhwc.permute(0, 3, 1, 2).contiguous()).t
    h = F.relu(F.conv2d(x_nhwc.permute(0, 3, 1, 2), K.permute(3, 2, 0, 1), kb))
    h = F.batch_norm(h, mean, var, gamma, beta, False, 0.0, 1e-3)
    h = F.max_pool2d(h, 2).permute(0, 2, 3, 1).reshape(3, -1)                    # Keras flattens NHWC
    assert torch.allclose(got, F.softmax(h @ W + wb, -1), atol=1e-4)


def test_keras_lstm_gate_order_and_npz(tmp_path):
    g = torch.Generator().manual_seed(2)
    nin, nh = 3, 4
    Wk, Uk, bk = torch.randn(nin, 4 * nh, generator=g) * 0.4, torch.randn(nh, 4 * nh, generator=g) * 0.4, torch.randn(4 * nh, generator=g) * 0.1
    Wd, bd = torch.randn(nh, 2, generator=g), torch.randn(2, generator=g)
    layers = [{"class_name": "LSTM", "config": {"name": "lstm", "units": nh, "activation": "tanh", "recurrent_activation": "sigmoid", "return_sequences": False,
                                                "batch_input_shape": [None, 6, nin]}},
              {"class_name": "Dense", "config": {"name": "out", "units": 2, "activation": "linear"}}]
    p = tmp_path / "w.npz"
    np.savez(p, **{"lstm/0": Wk.numpy(), "lstm/1": Uk.numpy(), "lstm/2": bk.numpy(), "out/0": Wd.numpy(), "out/1": bd.numpy()})
    net = KerasModelImport.importKerasSequentialModelAndWeights(_seq_json(layers, "mse"), str(p))
    x = torch.randn(2, 6, nin, generator=g)                                       # Keras [N, T, C]
    got = net.output(x.permute(0, 2, 1).contiguous()).t
    h, c = torch.zeros(2, nh), torch.zeros(2, nh)
    for t in range(6):
        z = x[:, t] @ Wk + h @ Uk + bk
        i, f, cc, o = z.chunk(4, 1)
        c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(cc)
        h = torch.sigmoid(o) * torch.tanh(c)
    assert torch.allclose(got, h @ Wd + bd, atol=1e-5)


def test_keras_functional_residual_and_errors():
    g = torch.Generator().manual_seed(3)
    W1, b1, W2, b2 = torch.randn(4, 4, generator=g), torch.randn(4, generator=g), torch.randn(8, 3, generator=g), torch.randn(3, generator=g)
    cfg = {"class_name": "Functional", "config": {"name": "m", "layers": [
        {"class_name": "InputLayer", "name": "inp", "config": {"name": "inp", "batch_input_shape": [None, 4]}, "inbound_nodes": []},
        {"class_name": "Dense", "name": "d1", "config": {"name": "d1", "units": 4, "activation": "tanh"}, "inbound_nodes": [[["inp", 0, 0, {}]]]},
        {"class_name": "Add", "name": "add", "config": {"name": "add"}, "inbound_nodes": [[["d1", 0, 0, {}], ["inp", 0, 0, {}]]]},
        {"class_name": "Concatenate", "name": "cat", "config": {"name": "cat", "axis": -1}, "inbound_nodes": [[["add", 0, 0, {}], ["inp", 0, 0, {}]]]},
        {"class_name": "Dense", "name": "out", "config": {"name": "out", "units": 3, "activation": "softmax"}, "inbound_nodes": [[["cat", 0, 0, {}]]]}],
        "input_layers": [["inp", 0, 0]], "output_layers": [["out", 0, 0]]}}
    net = KerasModelImport.importKerasModelAndWeights(json.dumps(cfg), {"d1": [W1.numpy(), b1.numpy()], "out": [W2.numpy(), b2.numpy()]}, loss="MCXENT")
    x = torch.randn(5, 4, generator=g)
    got = net.output(x)
    got = (got[0] if isinstance(got, (list, tuple)) else got).t
    h = torch.tanh(x @ W1 + b1) + x
    assert torch.allclose(got, F.softmax(torch.cat([h, x], 1) @ W2 + b2, -1), atol=1e-5)
    with pytest.raises(UnsupportedKerasConfigurationException, match="Lambda"):
        KerasModelImport.importKerasSequentialModelAndWeights(_seq_json([{"class_name": "Lambda", "config": {"name": "l", "batch_input_shape": [None, 3]}}]))
    with pytest.raises(FileNotFoundError):                  # HDF5 weights go through importers/hdf5.py (tests/test_hdf5_keras.py)
        KerasModelImport.importKerasSequentialModelAndWeights(_seq_json([{"class_name": "Dense", "config": {"name": "d", "units": 2, "batch_input_shape": [None, 3]}}]), "weights.h5")


def _c(name, arr):
    return tf_node(name, "Const", value=np.asarray(arr))


def test_tensorflow_while_loop_control_flow_import():
    """A TensorFlow 1.x while loop (Enter / Merge / LoopCond / Switch / Identity / NextIteration / Exit, with the back edge
    referring to a node that comes later in the file):  i = 0, acc = x;  while i < n: acc = acc * 2 + i; i += 1."""
    f32, i32 = np.float32, np.int32
    graph = b"".join([
        tf_node("x", "Placeholder", dtype=("dtype", 1), shape=("shape", [3])),
        _c("zero", np.asarray(0, i32)), _c("n", np.asarray(5, i32)), _c("one", np.asarray(1, i32)), _c("two", np.asarray(2.0, f32)),
        tf_node("while/Enter", "Enter", ["zero"], frame_name="while/ctx", is_constant=False),
        tf_node("while/Enter_1", "Enter", ["x"], frame_name="while/ctx", is_constant=False),
        tf_node("while/n", "Enter", ["n"], frame_name="while/ctx", is_constant=True),
        tf_node("while/one", "Enter", ["one"], frame_name="while/ctx", is_constant=True),
        tf_node("while/two", "Enter", ["two"], frame_name="while/ctx", is_constant=True),
        tf_node("while/Merge", "Merge", ["while/Enter", "while/NextIteration"]),
        tf_node("while/Merge_1", "Merge", ["while/Enter_1", "while/NextIteration_1"]),
        tf_node("while/Less", "Less", ["while/Merge", "while/n"]),
        tf_node("while/LoopCond", "LoopCond", ["while/Less"]),
        tf_node("while/Switch", "Switch", ["while/Merge", "while/LoopCond"]),
        tf_node("while/Switch_1", "Switch", ["while/Merge_1", "while/LoopCond"]),
        tf_node("while/Identity", "Identity", ["while/Switch:1"]),
        tf_node("while/Identity_1", "Identity", ["while/Switch_1:1"]),
        tf_node("while/mul", "Mul", ["while/Identity_1", "while/two"]),
        tf_node("while/cast", "Cast", ["while/Identity"], DstT=("dtype", 1)),
        tf_node("while/acc", "AddV2", ["while/mul", "while/cast"]),
        tf_node("while/inc", "AddV2", ["while/Identity", "while/one"]),
        tf_node("while/NextIteration", "NextIteration", ["while/inc"]),
        tf_node("while/NextIteration_1", "NextIteration", ["while/acc"]),
        tf_node("while/Exit", "Exit", ["while/Switch"]),
        tf_node("while/Exit_1", "Exit", ["while/Switch_1:0"]),
        tf_node("out", "Identity", ["while/Exit_1"])])
    imp = TensorflowFrameworkImporter()
    sd = imp.runImport(graph)
    x = torch.tensor([1.0, -2.0, 0.5])
    res = sd.output({"x": x}, "out", "while/Exit")
    acc = x.clone()
    for i in range(5):
        acc = acc * 2 + i
    assert torch.allclose(res["out"].t, acc) and int(res["while/Exit"].t) == 5
    # the imported loop survives a FlatBuffers round trip
    from deeplearning4j_b200.samediff.core import SameDiff
    back = SameDiff.fromFlatBuffers(sd.asFlatBuffers())
    assert torch.allclose(back.output({"x": x}, "out")["out"].t, acc)


def test_tensorflow_generic_rules_against_torch():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 4, 6, 3, generator=g)
    f32, i32 = np.float32, np.int32
    K = (torch.randn(3, 3, 5, 3, generator=g) * 0.2)                                  # HWIO with I = output channels of the transpose
    graph = b"".join([
        tf_node("x", "Placeholder", dtype=("dtype", 1), shape=("shape", [2, 4, 6, 3])),
        _c("begin", np.asarray([0, 1, 0, 0], i32)), _c("size", np.asarray([-1, 2, 3, -1], i32)),
        tf_node("sl", "Slice", ["x", "begin", "size"]),
        _c("b", np.asarray([0, 0, 1, 0], i32)), _c("e", np.asarray([0, 0, 6, 0], i32)), _c("s", np.asarray([1, 1, 2, 1], i32)),
        tf_node("ss", "StridedSlice", ["x", "b", "e", "s"], begin_mask=11, end_mask=11, shrink_axis_mask=0),
        _c("axis1", np.asarray(1, i32)), tf_node("sp", "Split", ["axis1", "x"], num_split=2),
        tf_node("spsum", "AddV2", ["sp", "sp:1"]),
        _c("k", np.asarray(2, i32)), tf_node("top", "TopKV2", ["x", "k"], sorted=True),
        _c("size2", np.asarray([8, 9], i32)), tf_node("rb", "ResizeBilinear", ["x", "size2"], align_corners=False, half_pixel_centers=True),
        tf_node("rn", "ResizeNearestNeighbor", ["x", "size2"], align_corners=False, half_pixel_centers=False),
        tf_node("s2d", "SpaceToDepth", ["x"], block_size=2, data_format="NHWC"), tf_node("d2s", "DepthToSpace", ["s2d"], block_size=2, data_format="NHWC"),
        _c("pads", np.asarray([[0, 0], [1, 2], [2, 1], [0, 0]], i32)), tf_node("mp", "MirrorPad", ["x", "pads"], mode="REFLECT"),
        tf_node("sp2", "MirrorPad", ["x", "pads"], mode="SYMMETRIC"),
        _c("lo", np.asarray(-0.5, f32)), _c("hi", np.asarray(0.25, f32)), tf_node("clip", "ClipByValue", ["x", "lo", "hi"]),
        tf_node("gt", "Greater", ["x", "hi"]), tf_node("sel", "SelectV2", ["gt", "x", "clip"]),
        _c("ax3", np.asarray(3, i32)), tf_node("cs", "Cumsum", ["x", "ax3"], exclusive=True, reverse=True),
        _c("idx", np.asarray([2, 0], i32)), _c("ax2", np.asarray(2, i32)), tf_node("ga", "GatherV2", ["x", "idx", "ax2"], batch_dims=0),
        _c("oshape", np.asarray([2, 8, 12, 5], i32)), _c("K", K.numpy()),
        tf_node("dc", "Conv2DBackpropInput", ["oshape", "K", "x"], strides=[1, 2, 2, 1], padding="SAME", data_format="NHWC"),
        tf_node("red", "Mean", ["x", "ax_dyn"], keep_dims=True), tf_node("ax_dyn", "Identity", ["ax3"]),
    ])
    # "red" reads "ax_dyn" which comes later in the file: a forward reference outside a loop is an error, so move it
    graph = graph.replace(tf_node("red", "Mean", ["x", "ax_dyn"], keep_dims=True) + tf_node("ax_dyn", "Identity", ["ax3"]),
                          tf_node("ax_dyn", "Identity", ["ax3"]) + tf_node("red", "Mean", ["x", "ax_dyn"], keep_dims=True))
    sd = TensorflowFrameworkImporter().runImport(graph)
    names = ["sl", "ss", "spsum", "top", "top:1", "rb", "rn", "d2s", "mp", "sp2", "sel", "cs", "ga", "dc", "red"]
    r = sd.output({"x": x}, *[n for n in names if ":" not in n])
    assert torch.equal(r["sl"].t, x[:, 1:3, 0:3]) and torch.equal(r["ss"].t, x[:, :, 1:6:2])
    assert torch.equal(r["spsum"].t, x[:, :2] + x[:, 2:])
    assert torch.equal(r["top"].t, torch.topk(x, 2).values)
    assert torch.allclose(r["rb"].t, F.interpolate(x.permute(0, 3, 1, 2), size=(8, 9), mode="bilinear", align_corners=False).permute(0, 2, 3, 1), atol=1e-6)
    ih, iw = (torch.arange(8) * (4 / 8)).floor().long(), (torch.arange(9) * (6 / 9)).floor().long()
    assert torch.equal(r["rn"].t, x[:, ih][:, :, iw])
    assert torch.equal(r["d2s"].t, x)
    assert torch.equal(r["mp"].t, F.pad(x.permute(0, 3, 1, 2), (2, 1, 1, 2), mode="reflect").permute(0, 2, 3, 1))
    assert torch.equal(r["sp2"].t[:, 0], x[:, 0][:, [1, 0, *range(6), 5]])                        # symmetric: border repeated
    assert torch.equal(r["sel"].t, torch.where(x > 0.25, x, x.clamp(-0.5, 0.25)))
    assert torch.allclose(r["cs"].t, x.flip(3).cumsum(3).flip(3) - x, atol=1e-6)
    assert torch.equal(r["ga"].t, x[:, :, [2, 0]])
    ref = F.conv_transpose2d(x.permute(0, 3, 1, 2), K.permute(3, 2, 0, 1), stride=2, padding=1, output_padding=1).permute(0, 2, 3, 1)
    assert tuple(r["dc"].t.shape) == (2, 8, 12, 5)
    # SAME padding of the transposed convolution: total padding k - s = 1, taken from the start (0) and the end (1)
    full = F.conv_transpose2d(x.permute(0, 3, 1, 2), K.permute(3, 2, 0, 1), stride=2).permute(0, 2, 3, 1)
    assert torch.allclose(r["dc"].t, full[:, 0:8, 0:12], atol=1e-5) and ref is not None
    assert torch.allclose(r["red"].t, x.mean(3, keepdim=True), atol=1e-6)
    assert len(TensorflowFrameworkImporter.supportedOps()) >= 150


def test_tensorflow_spatial_scatter_and_3d_rules_by_their_definitions():
    """Rules added for the less common GraphDef ops, each checked against the TensorFlow definition of the op
    written out in plain torch (tensorflow/core/ops: array_ops.cc, nn_ops.cc, image_ops.cc)."""
    from deeplearning4j_b200.importers.tf_import import _tf_ops
    T = {k: v[0] for k, v in _tf_ops().items()}
    g = torch.Generator().manual_seed(5)

    x = torch.randn(5, 6, generator=g)
    got = T["MatrixBandPart"](x, torch.tensor(1), torch.tensor(-1))
    assert torch.equal(got, torch.triu(x, -1))
    got = T["MatrixBandPart"](x, torch.tensor(0), torch.tensor(2))
    assert torch.equal(got, torch.triu(x) - torch.triu(x, 3))

    idx = torch.tensor([[0, 1], [2, 3], [0, 1]])
    upd = torch.tensor([1.0, 2.0, 4.0])
    out = T["ScatterNd"](idx, upd, torch.tensor([3, 4]))
    ref = torch.zeros(3, 4); ref[0, 1] = 5.0; ref[2, 3] = 2.0
    assert torch.equal(out, ref)
    rows = T["ScatterNd"](torch.tensor([[1]]), torch.ones(1, 4), torch.tensor([3, 4]))
    assert torch.equal(rows[1], torch.ones(4)) and rows.sum() == 4

    # space-to-batch with block 2 is the inverse pixel shuffle with the block index moved into the batch
    x = torch.arange(1 * 4 * 6 * 2, dtype=torch.float32).reshape(1, 4, 6, 2)
    y = T["SpaceToBatchND"](x, torch.tensor([2, 2]), torch.zeros(2, 2, dtype=torch.int64))
    assert tuple(y.shape) == (4, 2, 3, 2)
    for bi in range(2):
        for bj in range(2):
            assert torch.equal(y[bi * 2 + bj, :, :, :], x[0, bi::2, bj::2, :])
    back = T["BatchToSpaceND"](y, torch.tensor([2, 2]), torch.zeros(2, 2, dtype=torch.int64))
    assert torch.equal(back, x)
    # padding on the way in, the same crops on the way out
    x = torch.randn(2, 3, 5, 1, generator=g)
    pad = torch.tensor([[1, 0], [0, 1]])
    y = T["SpaceToBatchND"](x, torch.tensor([2, 2]), pad)
    assert tuple(y.shape) == (8, 2, 3, 1)
    assert torch.equal(T["BatchToSpaceND"](y, torch.tensor([2, 2]), pad), x)

    x = torch.randn(2, 5, 6, 7, 3, generator=g)
    w = torch.randn(3, 3, 3, 3, 4, generator=g)
    y = T["Conv3D"](x, w, strides=[1, 1, 1, 1, 1], padding=b"SAME")
    ref = F.conv3d(x.permute(0, 4, 1, 2, 3), w.permute(4, 3, 0, 1, 2), padding=1).permute(0, 2, 3, 4, 1)
    assert torch.allclose(y, ref, atol=1e-5)
    y = T["Conv3D"](x, w, strides=[1, 2, 2, 2, 1], padding=b"VALID")
    ref = F.conv3d(x.permute(0, 4, 1, 2, 3), w.permute(4, 3, 0, 1, 2), stride=2).permute(0, 2, 3, 4, 1)
    assert torch.allclose(y, ref, atol=1e-5)
    y = T["MaxPool3D"](x, ksize=[1, 2, 2, 2, 1], strides=[1, 2, 2, 2, 1], padding=b"VALID")
    assert torch.equal(y, F.max_pool3d(x.permute(0, 4, 1, 2, 3), 2, 2).permute(0, 2, 3, 4, 1))
    y = T["MaxPool3D"](x, ksize=[1, 2, 2, 2, 1], strides=[1, 2, 2, 2, 1], padding=b"SAME")
    assert tuple(y.shape) == (2, 3, 3, 4, 3)
    assert torch.equal(y[:, 2, :, 3, :], x[:, 4, :, 6, :].reshape(2, 3, 2, 3).amax(2))   # the ragged corner sees only real elements
    y = T["AvgPool3D"](x, ksize=[1, 2, 2, 2, 1], strides=[1, 2, 2, 2, 1], padding=b"SAME")
    assert torch.allclose(y[:, 2, :, 3, :], x[:, 4, :, 6, :].reshape(2, 3, 2, 3).mean(2), atol=1e-6)

    a, b = T["ShapeN"](torch.zeros(2, 3), torch.zeros(4))
    assert a.tolist() == [2, 3] and b.tolist() == [4]
    r = T["RandomUniform"](torch.tensor([3, 5]))
    assert tuple(r.shape) == (3, 5) and float(r.min()) >= 0 and float(r.max()) < 1
    c = torch.tensor(True)
    assert T["Assert"](c, torch.zeros(1)) is c

    boxes = torch.tensor([[0, 0, 1, 1], [0, 0.1, 1, 1.1], [0, -0.1, 1, 0.9], [0, 10, 1, 11], [0, 10.1, 1, 11.1], [0, 100, 1, 101]], dtype=torch.float32)
    scores = torch.tensor([0.9, 0.75, 0.6, 0.95, 0.5, 0.3])
    sel = T["NonMaxSuppressionV3"](boxes, scores, torch.tensor(3), torch.tensor(0.5), torch.tensor(0.0))
    assert sel.tolist() == [3, 0, 5]
    sel = T["NonMaxSuppressionV3"](boxes, scores, torch.tensor(6), torch.tensor(0.5), torch.tensor(0.4))
    assert sel.tolist() == [3, 0]


def test_tensorflow_second_operator_table_by_definitions():
    """Special functions, segment / scatter / partition ops, linear algebra, image ops and older spellings: each against the
    TensorFlow definition written out in plain torch / numpy (tensorflow/core/ops/{math,array,linalg,image,nn}_ops.cc)."""
    from deeplearning4j_b200.importers.tf_import import _tf_ops
    T = {k: v[0] for k, v in _tf_ops().items()}
    g = torch.Generator().manual_seed(11)
    R = lambda *s: torch.randn(*s, generator=g)

    x = R(7).abs() + 0.5
    assert torch.allclose(T["Lgamma"](x), torch.lgamma(x)) and torch.allclose(T["Digamma"](x), torch.digamma(x))
    assert torch.allclose(T["Igamma"](x, x + 1) + T["Igammac"](x, x + 1), torch.ones(7), atol=1e-6)
    assert torch.allclose(T["Polygamma"](torch.tensor(1), x), torch.special.polygamma(1, x))
    assert T["Xdivy"](torch.tensor([0.0, 2.0]), torch.tensor([0.0, 4.0])).tolist() == [0.0, 0.5]
    assert T["DivNoNan"](torch.tensor([1.0, 2.0]), torch.tensor([0.0, 4.0])).tolist() == [0.0, 0.5]
    assert T["TruncateMod"](torch.tensor([-7, 7]), torch.tensor([3, -3])).tolist() == [-1, 1]
    assert T["LeftShift"](torch.tensor([1, 3]), torch.tensor([2, 1])).tolist() == [4, 6] and T["BitwiseXor"](torch.tensor([6]), torch.tensor([3])).tolist() == [5]
    assert T["BroadcastArgs"](torch.tensor([3, 1]), torch.tensor([1, 4])).tolist() == [3, 4]
    assert torch.equal(T["Concat"](torch.tensor(1), torch.ones(2, 1), torch.zeros(2, 2)), torch.tensor([[1.0, 0, 0], [1.0, 0, 0]]))
    d = T["Diag"](torch.tensor([[1.0, 2.0], [3.0, 4.0]]))
    assert d.shape == (2, 2, 2, 2) and d[1, 0, 1, 0] == 3 and d[0, 1, 1, 0] == 0 and torch.equal(T["DiagPart"](d), torch.tensor([[1.0, 2.0], [3.0, 4.0]]))
    m = R(3, 4, 4)
    assert torch.equal(T["MatrixSetDiag"](m, torch.ones(3, 4)).diagonal(0, -2, -1), torch.ones(3, 4))
    spd = m @ m.transpose(1, 2) + 4 * torch.eye(4)
    L = T["Cholesky"](spd)
    assert torch.allclose(L @ L.transpose(1, 2), spd, atol=1e-4)
    b = R(3, 4, 2)
    assert torch.allclose(spd @ T["MatrixSolve"](spd, b), b, atol=1e-3)
    assert torch.allclose(L @ T["MatrixTriangularSolve"](L, b, lower=True), b, atol=1e-4)
    assert torch.allclose(L.transpose(1, 2) @ T["MatrixTriangularSolve"](L, b, lower=True, adjoint=True), b, atol=1e-4)
    sign, logdet = T["LogMatrixDeterminant"](spd)
    assert torch.allclose(sign * logdet.exp(), T["MatrixDeterminant"](spd), rtol=1e-4)
    s, u, v = T["Svd"](m)
    assert torch.allclose(u @ torch.diag_embed(s) @ v.transpose(1, 2), m, atol=1e-4)
    lu, perm = T["Lu"](m[0])
    Lm, Um = torch.tril(lu, -1) + torch.eye(4), torch.triu(lu)
    assert torch.allclose(Lm @ Um, m[0][perm.long()], atol=1e-5)                       # TensorFlow: P applied to the rows of the input

    data = torch.tensor([[1.0, 2], [3, 4], [5, 6], [7, 8]])
    ids = torch.tensor([0, 0, 2, 2])
    assert T["SegmentSum"](data, ids).tolist() == [[4, 6], [0, 0], [12, 14]] and T["SegmentMean"](data, ids).tolist() == [[2, 3], [0, 0], [6, 7]]
    assert T["SegmentMax"](data, ids).tolist() == [[3, 4], [0, 0], [7, 8]] and T["SegmentProd"](data, ids).tolist() == [[3, 8], [1, 1], [35, 48]]
    um = T["UnsortedSegmentMax"](data, torch.tensor([1, -1, 1, 0]), torch.tensor(3))
    assert um[:2].tolist() == [[7, 8], [5, 6]] and um[2, 0] == torch.finfo(torch.float32).min
    assert T["UnsortedSegmentSum"](data, torch.tensor([1, -1, 1, 0]), torch.tensor(2)).tolist() == [[7, 8], [6, 8]]
    idx = torch.tensor([[0, 1], [3, 0]])
    assert T["TensorScatterAdd"](data, idx, torch.tensor([10.0, 20]))[0].tolist() == [1, 12] and T["TensorScatterUpdate"](data, idx, torch.tensor([10.0, 20]))[3, 0] == 20
    assert T["TensorScatterSub"](data, torch.tensor([[1]]), torch.tensor([[1.0, 1]]))[1].tolist() == [2, 3]
    p0, p1 = T["DynamicPartition"](data, torch.tensor([1, 0, 1, 0]), num_partitions=2)
    assert p0.tolist() == [[3, 4], [7, 8]] and p1.tolist() == [[1, 2], [5, 6]]
    assert torch.equal(T["DynamicStitch"](torch.tensor([1, 3]), torch.tensor([0, 2]), p0, p1), data)

    fq = T["FakeQuantWithMinMaxArgs"](torch.tensor([-7.0, -0.02, 0.0, 0.03, 2.9, 9.0]), min=-6.0, max=6.0, num_bits=8)
    step = 12.0 / 255
    assert torch.allclose(fq[1:4] / step, torch.round(fq[1:4] / step), atol=1e-4) and fq[2] == 0 and abs(float(fq[0]) + 6) < step and abs(float(fq[5]) - 6) < step
    assert T["InTopKV2"](torch.tensor([[0.1, 0.9, 0.5], [0.3, 0.2, 0.1]]), torch.tensor([2, 2]), torch.tensor(2)).tolist() == [True, False]
    assert T["InvertPermutation"](torch.tensor([2, 0, 1])).tolist() == [1, 2, 0]
    assert T["LinSpace"](torch.tensor(1.0), torch.tensor(2.0), torch.tensor(5)).tolist() == [1.0, 1.25, 1.5, 1.75, 2.0]
    o, i = T["ListDiff"](torch.tensor([1, 2, 3, 4, 5, 6]), torch.tensor([1, 3, 5]))
    assert o.tolist() == [2, 4, 6] and i.tolist() == [1, 3, 5]
    assert T["HistogramFixedWidth"](torch.tensor([-1.0, 0.0, 1.5, 2.0, 5.0, 15.0]), torch.tensor([0.0, 5.0]), torch.tensor(5)).tolist() == [2, 1, 1, 0, 2]
    assert T["Bincount"](torch.tensor([1, 1, 3]), torch.tensor(5), torch.tensor([])).tolist() == [0, 2, 0, 1, 0]
    u_, ix_, cnt = T["UniqueWithCounts"](torch.tensor([4, 1, 4, 7, 1, 4]))
    assert u_.tolist() == [4, 1, 7] and ix_.tolist() == [0, 1, 0, 2, 1, 0] and cnt.tolist() == [3, 2, 1]
    assert T["NthElement"](torch.tensor([[5, 1, 3], [2, 9, 4]]), torch.tensor(1)).tolist() == [3, 4]
    assert torch.allclose(T["ClipByNorm"](torch.tensor([3.0, 4.0]), torch.tensor(1.0)), torch.tensor([0.6, 0.8]))
    assert T["Roll"](torch.arange(5), torch.tensor(2), torch.tensor(0)).tolist() == [3, 4, 0, 1, 2]
    assert T["Reverse"](torch.arange(6).reshape(2, 3), torch.tensor([False, True])).tolist() == [[2, 1, 0], [5, 4, 3]]
    rs = T["ReverseSequence"](torch.arange(8).reshape(2, 4), torch.tensor([3, 2]), seq_dim=1, batch_dim=0)
    assert rs.tolist() == [[2, 1, 0, 3], [5, 4, 6, 7]]
    assert T["RandomUniformInt"](torch.tensor([50]), torch.tensor(3), torch.tensor(6)).unique().tolist() == [3, 4, 5]
    assert tuple(T["Multinomial"](R(2, 5), torch.tensor(7)).shape) == (2, 7) and float(T["TruncatedNormal"](torch.tensor([1000])).abs().max()) <= 2.0

    img = R(2, 6, 6, 3)
    y, am = T["MaxPoolWithArgmax"](img, ksize=[1, 2, 2, 1], strides=[1, 2, 2, 1], padding=b"VALID")
    assert torch.equal(y, F.max_pool2d(img.permute(0, 3, 1, 2), 2).permute(0, 2, 3, 1))
    assert torch.equal(img[0].reshape(-1)[am[0].reshape(-1)], y[0].reshape(-1))          # flat (h, w, c) index into one image
    pt = T["ExtractImagePatches"](img, ksizes=[1, 2, 2, 1], strides=[1, 2, 2, 1], rates=[1, 1, 1, 1], padding=b"VALID")
    assert pt.shape == (2, 3, 3, 12) and torch.equal(pt[1, 2, 1], img[1, 4:6, 2:4, :].reshape(-1))
    dl = T["Dilation2D"](img, torch.zeros(2, 2, 3), strides=[1, 1, 1, 1], rates=[1, 1, 1, 1], padding=b"VALID")
    assert torch.equal(dl, F.max_pool2d(img.permute(0, 3, 1, 2), 2, 1).permute(0, 2, 3, 1))
    rgb = torch.rand(4, 5, 3, generator=g)
    assert torch.allclose(T["HSVToRGB"](T["RGBToHSV"](rgb)), rgb, atol=1e-5)
    assert T["RGBToHSV"](torch.tensor([[0.0, 1.0, 0.0]]))[0].tolist() == pytest.approx([1 / 3, 1.0, 1.0])
    assert torch.allclose(T["AdjustHue"](rgb, 1.0), rgb, atol=1e-5) and torch.allclose(T["AdjustSaturation"](rgb, 0.0), rgb.max(-1, keepdim=True).values.expand_as(rgb), atol=1e-6)
    ac = T["AdjustContrastV2"](img, 2.0)
    assert torch.allclose(ac.mean((1, 2)), img.mean((1, 2)), atol=1e-5) and torch.allclose(ac - ac.mean((1, 2), keepdim=True), 2 * (img - img.mean((1, 2), keepdim=True)), atol=1e-5)
    cr = T["CropAndResize"](img, torch.tensor([[0.0, 0.0, 1.0, 1.0], [0.2, 0.2, 0.6, 0.6]]), torch.tensor([1, 0]), torch.tensor([6, 6]))
    assert torch.allclose(cr[0], img[1], atol=1e-6) and cr.shape == (2, 6, 6, 3)
    cr = T["CropAndResize"](img, torch.tensor([[0.0, 0.0, 0.4, 0.4]]), torch.tensor([0]), torch.tensor([3, 3]))       # lands on the pixel centres 0, 1, 2
    assert torch.allclose(cr[0], img[0, :3, :3], atol=1e-6)
    assert T["ResizeArea"](img, torch.tensor([3, 3])).shape == (2, 3, 3, 3) and torch.allclose(T["ResizeArea"](img, torch.tensor([3, 3])), F.avg_pool2d(img.permute(0, 3, 1, 2), 2).permute(0, 2, 3, 1), atol=1e-6)
    boxes = torch.tensor([[0, 0, 1, 1], [0, 0.05, 1, 1.05], [0, 3, 1, 4]], dtype=torch.float32)
    sel, n = T["NonMaxSuppressionV4"](boxes, torch.tensor([0.9, 0.8, 0.7]), torch.tensor(3), torch.tensor(0.5), torch.tensor(0.0), pad_to_max_output_size=True)
    assert sel.tolist() == [0, 2, 0] and int(n) == 2
    sel, sc, n = T["NonMaxSuppressionV5"](boxes, torch.tensor([0.9, 0.8, 0.7]), torch.tensor(3), torch.tensor(0.5), torch.tensor(0.0), torch.tensor(0.0))
    assert sel.tolist() == [0, 2] and sc.tolist() == pytest.approx([0.9, 0.7])
    db = T["DrawBoundingBoxes"](torch.zeros(1, 5, 5, 3), torch.tensor([[[0.0, 0.0, 1.0, 1.0]]]), torch.tensor([[1.0, 0.0, 0.0]]))
    assert db[0, 0, 2].tolist() == [1, 0, 0] and db[0, 2, 0].tolist() == [1, 0, 0] and db[0, 2, 2].tolist() == [0, 0, 0]

    # gradients of the convolutions against autograd
    x3 = R(1, 4, 5, 5, 2).requires_grad_(True)
    w3 = R(2, 2, 2, 2, 3)
    y3 = F.conv3d(x3.permute(0, 4, 1, 2, 3), w3.permute(4, 3, 0, 1, 2), stride=(1, 2, 1)).permute(0, 2, 3, 4, 1)
    dy3 = R(*y3.shape)
    y3.backward(dy3)
    got = T["Conv3DBackpropInputV2"](torch.tensor([1, 4, 5, 5, 2]), w3, dy3, strides=[1, 1, 2, 1, 1], padding=b"VALID")
    assert torch.allclose(got, x3.grad, atol=1e-5)
    x2 = R(2, 6, 7, 3)
    w2 = R(3, 3, 3, 4).requires_grad_(True)
    xp = F.pad(x2.permute(0, 3, 1, 2), (1, 1, 0, 1))                                  # SAME for 6x7, k 3, stride 2: rows (0, 1), columns (1, 1)
    y2 = F.conv2d(xp, w2.permute(3, 2, 0, 1), stride=2).permute(0, 2, 3, 1)
    dy2 = R(*y2.shape)
    y2.backward(dy2)
    got = T["Conv2DBackpropFilter"](x2, torch.tensor([3, 3, 3, 4]), dy2, strides=[1, 2, 2, 1], padding=b"SAME")
    assert torch.allclose(got, w2.grad, atol=1e-4)
