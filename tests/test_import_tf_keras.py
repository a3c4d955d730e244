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
    with pytest.raises(UnsupportedKerasConfigurationException, match="h5py"):
        KerasModelImport.importKerasSequentialModelAndWeights(_seq_json([{"class_name": "Dense", "config": {"name": "d", "units": 2, "batch_input_shape": [None, 3]}}]), "weights.h5")
