"""Keras layer mappers beyond the basic set (``deeplearning4j-modelimport/.../keras/layers/**``): each imported network
is compared with the layer's definition written out in plain torch on channels-last data."""
import json

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from deeplearning4j_b200 import nn
from deeplearning4j_b200.importers import KerasModelImport, UnsupportedKerasConfigurationException

RNG = np.random.default_rng(7)


def L(cls, **cfg):
    return {"class_name": cls, "config": cfg}


def seq(layers):
    return json.dumps({"class_name": "Sequential", "config": {"layers": layers}})


def arr(*shape, scale=0.3):
    return (RNG.normal(size=shape) * scale).astype("f4")


def out(net, x):
    y = net.output(x)
    y = y[0] if isinstance(y, (list, tuple)) else y
    return torch.as_tensor(np.asarray(y.numpy() if hasattr(y, "numpy") else y))


def t(a):
    return torch.from_numpy(np.asarray(a))


def test_conv3d_pool3d_flatten_dense():
    layers = [L("Conv3D", name="c3", filters=4, kernel_size=[2, 2, 2], strides=[1, 1, 1], padding="valid", activation="relu", batch_input_shape=[None, 4, 5, 6, 2]),
              L("ZeroPadding3D", name="zp", padding=[[1, 0], [0, 1], [1, 1]]),
              L("MaxPooling3D", name="p3", pool_size=[2, 2, 2], padding="valid"),
              L("UpSampling3D", name="up", size=[1, 2, 1]),
              L("Cropping3D", name="cr", cropping=[[0, 0], [1, 0], [0, 1]]),
              L("Flatten", name="fl"),
              L("Dense", name="d", units=3, activation="softmax")]
    w = {"c3": [arr(2, 2, 2, 2, 4), arr(4)], "d": [arr(2 * 3 * 2 * 4, 3), arr(3)]}
    net = KerasModelImport.importKerasSequentialModelAndWeights(seq(layers), w, loss="MCXENT")
    assert net.kerasInputLayout == "NDHWC"
    x = torch.randn(2, 4, 5, 6, 2)
    r = F.conv3d(x.permute(0, 4, 1, 2, 3), t(w["c3"][0]).permute(4, 3, 0, 1, 2), t(w["c3"][1])).relu()       # 3, 4, 5
    r = F.pad(r, (1, 1, 0, 1, 1, 0))                                                                           # 4, 5, 7
    r = F.max_pool3d(r, 2)                                                                                     # 2, 2, 3
    r = r.repeat_interleave(2, 3)                                                                              # 2, 4, 3
    r = r[:, :, :, 1:, :2]                                                                                     # 2, 3, 2
    r = r.permute(0, 2, 3, 4, 1).reshape(2, -1)                                                                # Keras flattens channels last
    r = (r @ t(w["d"][0]) + t(w["d"][1])).softmax(-1)
    assert torch.allclose(out(net, x.permute(0, 4, 1, 2, 3).contiguous()), r, atol=1e-5)


def test_conv3d_transpose_and_global_pooling():
    layers = [L("Conv3DTranspose", name="dc", filters=3, kernel_size=[2, 2, 2], strides=[2, 2, 2], padding="valid", activation="linear", batch_input_shape=[None, 2, 3, 2, 2]),
              L("GlobalAveragePooling3D", name="gp")]
    w = {"dc": [arr(2, 2, 2, 3, 2), arr(3)]}
    net = KerasModelImport.importKerasSequentialModelAndWeights(seq(layers), w)
    x = torch.randn(2, 2, 3, 2, 2)
    r = F.conv_transpose3d(x.permute(0, 4, 1, 2, 3), t(w["dc"][0]).permute(4, 3, 0, 1, 2), t(w["dc"][1]), stride=2).mean((2, 3, 4))
    assert torch.allclose(out(net, x.permute(0, 4, 1, 2, 3).contiguous()), r, atol=1e-5)


def test_one_dimensional_padding_cropping_upsampling():
    layers = [L("ZeroPadding1D", name="zp", padding=[2, 1], batch_input_shape=[None, 5, 3]),
              L("UpSampling1D", name="up", size=2),
              L("Cropping1D", name="cr", cropping=[1, 3])]
    net = KerasModelImport.importKerasSequentialModelAndWeights(seq(layers))
    x = torch.randn(2, 5, 3)                                            # Keras [batch, steps, features]
    r = F.pad(x, (0, 0, 2, 1)).repeat_interleave(2, 1)[:, 1:-3]
    assert torch.allclose(out(net, x.permute(0, 2, 1).contiguous()).permute(0, 2, 1), r)


def test_reshape_and_permute_follow_the_channels_last_convention():
    layers = [L("Reshape", name="rs", target_shape=[4, 3, 2], batch_input_shape=[None, 24]),
              L("Conv2D", name="c", filters=2, kernel_size=[2, 2], padding="valid", activation="linear"),
              L("Permute", name="pm", dims=[2, 1, 3]),
              L("Reshape", name="rs2", target_shape=[-1, 2]),
              L("LSTM", name="l", units=3, activation="tanh", recurrent_activation="sigmoid", return_sequences=False)]
    w = {"c": [arr(2, 2, 2, 2), arr(2)], "l": [arr(2, 12), arr(3, 12), arr(12)]}
    net = KerasModelImport.importKerasSequentialModelAndWeights(seq(layers), w)
    x = torch.randn(3, 24)
    r = x.reshape(3, 4, 3, 2)
    r = F.conv2d(r.permute(0, 3, 1, 2), t(w["c"][0]).permute(3, 2, 0, 1), t(w["c"][1])).permute(0, 2, 3, 1)     # [3, 3, 2, 2]
    r = r.permute(0, 2, 1, 3).reshape(3, -1, 2)                                                                  # [3, 6, 2]
    W, U, b = (t(a) for a in w["l"])
    h = c = torch.zeros(3, 3)
    for s in range(r.shape[1]):
        z = r[:, s] @ W + h @ U + b
        i, f, g, o = z.chunk(4, -1)
        c = f.sigmoid() * c + i.sigmoid() * g.tanh()
        h = o.sigmoid() * c.tanh()
    assert torch.allclose(out(net, x), h, atol=1e-5)
    # the pre-processors survive the configuration's JSON form
    from deeplearning4j_b200.nn.conf.neuralnet import MultiLayerConfiguration
    again = MultiLayerConfiguration.fromJson(net.conf.toJson())
    assert again.inputPreProcessors.keys() == net.conf.inputPreProcessors.keys()
    assert all(again.inputPreProcessors[k] == v for k, v in net.conf.inputPreProcessors.items())


def test_bidirectional_lstm_and_time_distributed_dense():
    for merge, comb in (("concat", lambda a, b: torch.cat([a, b], -1)), ("sum", lambda a, b: a + b), ("ave", lambda a, b: 0.5 * (a + b)), ("mul", lambda a, b: a * b)):
        layers = [L("Bidirectional", name="bi", merge_mode=merge, batch_input_shape=[None, 5, 2],
                    layer=L("LSTM", name="inner", units=3, activation="tanh", recurrent_activation="sigmoid", return_sequences=True)),
                  L("TimeDistributed", name="td", layer=L("Dense", name="tdd", units=2, activation="tanh"))]
        n = 6 if merge == "concat" else 3
        w = {"bi": [arr(2, 12), arr(3, 12), arr(12), arr(2, 12), arr(3, 12), arr(12)], "td": [arr(n, 2), arr(2)]}
        net = KerasModelImport.importKerasSequentialModelAndWeights(seq(layers), w)
        x = torch.randn(2, 5, 2)

        def run(W, U, b, xs):
            h = c = torch.zeros(2, 3)
            hs = []
            for s in range(xs.shape[1]):
                i, f, g, o = (xs[:, s] @ W + h @ U + b).chunk(4, -1)
                c = f.sigmoid() * c + i.sigmoid() * g.tanh()
                h = o.sigmoid() * c.tanh()
                hs.append(h)
            return torch.stack(hs, 1)
        fw = run(*(t(a) for a in w["bi"][:3]), x)
        bw = run(*(t(a) for a in w["bi"][3:]), x.flip(1)).flip(1)
        r = (comb(fw, bw) @ t(w["td"][0]) + t(w["td"][1])).tanh()
        assert torch.allclose(out(net, x.permute(0, 2, 1).contiguous()).permute(0, 2, 1), r, atol=1e-5), merge


def test_masking_reaches_the_recurrent_layer():
    layers = [L("Masking", name="m", mask_value=0.0, batch_input_shape=[None, 4, 2]),
              L("SimpleRNN", name="r", units=3, activation="tanh", return_sequences=False)]
    w = {"r": [arr(2, 3), arr(3, 3), arr(3)]}
    net = KerasModelImport.importKerasSequentialModelAndWeights(seq(layers), w)
    assert type(net.conf.layers()[0]).__name__ == "MaskZeroLayer"
    x = torch.randn(2, 4, 2)
    x[0, 2:] = 0.0                                                      # example 0 ends after two steps
    W, U, b = (t(a) for a in w["r"])
    ref = []
    for e, steps in ((0, 2), (1, 4)):
        h = torch.zeros(3)
        for s in range(steps):
            h = (x[e, s] @ W + h @ U + b).tanh()
        ref.append(h)
    assert torch.allclose(out(net, x.permute(0, 2, 1).contiguous()), torch.stack(ref), atol=1e-5)


def test_prelu_shared_axes_noise_layers_and_parametrised_activations():
    layers = [L("Conv2D", name="c", filters=3, kernel_size=[1, 1], activation="linear", batch_input_shape=[None, 4, 5, 2]),
              L("PReLU", name="pr", shared_axes=[1, 2]),
              L("GaussianNoise", name="gn", stddev=0.5), L("GaussianDropout", name="gd", rate=0.3), L("AlphaDropout", name="ad", rate=0.2),
              L("SpatialDropout2D", name="sd", rate=0.4),
              L("ELU", name="elu", alpha=0.7), L("ThresholdedReLU", name="tr", theta=0.05)]
    w = {"c": [arr(1, 1, 2, 3), arr(3)], "pr": [np.asarray([[[0.1, 0.2, 0.3]]], dtype="f4")]}
    net = KerasModelImport.importKerasSequentialModelAndWeights(seq(layers), w)
    x = torch.randn(2, 4, 5, 2)
    r = F.conv2d(x.permute(0, 3, 1, 2), t(w["c"][0]).permute(3, 2, 0, 1), t(w["c"][1]))
    a = t(w["pr"][0]).reshape(1, 3, 1, 1)
    r = torch.where(r >= 0, r, a * r)
    r = F.elu(r, 0.7)
    r = torch.where(r > 0.05, r, torch.zeros_like(r))
    assert torch.allclose(out(net, x.permute(0, 3, 1, 2).contiguous()), r, atol=1e-5)       # the noise layers do nothing at inference
    kinds = [type(l.dropOut).__name__ for l in net.conf.layers()[2:6]]
    assert kinds == ["GaussianNoise", "GaussianDropout", "AlphaDropout", "SpatialDropout"]

    # full-shape PReLU: Keras keeps alpha as (h, w, c)
    layers = [L("PReLU", name="pr", batch_input_shape=[None, 2, 3, 2])]
    alpha = arr(2, 3, 2)
    net = KerasModelImport.importKerasSequentialModelAndWeights(seq(layers), {"pr": [alpha]})
    x = torch.randn(2, 2, 3, 2)
    assert torch.allclose(out(net, x.permute(0, 3, 1, 2).contiguous()).permute(0, 2, 3, 1), torch.where(x >= 0, x, t(alpha) * x), atol=1e-6)


def test_locally_connected_space_to_depth_lrn_and_repeat_vector():
    layers = [L("LocallyConnected2D", name="lc", filters=2, kernel_size=[2, 2], strides=[1, 1], padding="valid", activation="linear", use_bias=False,
                batch_input_shape=[None, 3, 4, 2])]
    w = {"lc": [arr(2 * 3, 2 * 2 * 2, 2)]}
    net = KerasModelImport.importKerasSequentialModelAndWeights(seq(layers), w)
    x = torch.randn(2, 3, 4, 2)
    ref = torch.zeros(2, 2, 3, 2)
    for i in range(2):
        for j in range(3):
            patch = x[:, i:i + 2, j:j + 2, :].reshape(2, -1)            # (kh, kw, in) feature order
            ref[:, i, j] = patch @ t(w["lc"][0])[i * 3 + j]
    assert torch.allclose(out(net, x.permute(0, 3, 1, 2).contiguous()).permute(0, 2, 3, 1), ref, atol=1e-5)

    layers = [L("LocallyConnected1D", name="lc", filters=2, kernel_size=[3], strides=[1], padding="valid", activation="tanh", use_bias=False, batch_input_shape=[None, 5, 2])]
    w = {"lc": [arr(3, 3 * 2, 2)]}
    net = KerasModelImport.importKerasSequentialModelAndWeights(seq(layers), w)
    x = torch.randn(2, 5, 2)
    ref = torch.stack([(x[:, s:s + 3].reshape(2, -1) @ t(w["lc"][0])[s]).tanh() for s in range(3)], 1)
    assert torch.allclose(out(net, x.permute(0, 2, 1).contiguous()).permute(0, 2, 1), ref, atol=1e-5)

    layers = [L("RepeatVector", name="rv", n=3, batch_input_shape=[None, 4])]
    net = KerasModelImport.importKerasSequentialModelAndWeights(seq(layers))
    x = torch.randn(2, 4)
    assert torch.allclose(out(net, x).permute(0, 2, 1), x[:, None, :].expand(2, 3, 4))

    layers = [L("LRN", name="lrn", n=3, k=1.5, alpha=1e-2, beta=0.6, batch_input_shape=[None, 2, 2, 5])]
    net = KerasModelImport.importKerasSequentialModelAndWeights(seq(layers))
    x = torch.randn(2, 2, 2, 5)
    sq = F.pad(x * x, (1, 1))
    win = sq[..., 0:5] + sq[..., 1:6] + sq[..., 2:7]
    assert torch.allclose(out(net, x.permute(0, 3, 1, 2).contiguous()).permute(0, 2, 3, 1), x / (1.5 + 1e-2 * win) ** 0.6, atol=1e-5)


def test_lambda_and_custom_layers_come_from_the_registries():
    layers = [L("Lambda", name="times_two", batch_input_shape=[None, 3]), L("Scale3", name="s3")]
    with pytest.raises(UnsupportedKerasConfigurationException, match="registerLambdaLayer"):
        KerasModelImport.importKerasSequentialModelAndWeights(seq(layers))

    class TimesTwo(nn.SameDiffLambdaLayer):
        def defineLayer(self, sd, x):
            return x * 2.0
    KerasModelImport.registerLambdaLayer("times_two", TimesTwo())
    KerasModelImport.registerCustomLayer("Scale3", lambda cfg: nn.ActivationLayer(nn.activations.ActivationLReLU(alpha=3.0), layerName=cfg["name"]))
    try:
        net = KerasModelImport.importKerasSequentialModelAndWeights(seq(layers))
        x = torch.tensor([[1.0, -1.0, 0.5]])
        assert torch.allclose(out(net, x), torch.tensor([[2.0, -6.0, 1.0]]))
    finally:
        KerasModelImport.clearLambdaLayers()


def test_functional_graph_with_reshape_vertex_and_masking():
    cfg = {"class_name": "Model", "config": {
        "name": "m", "input_layers": [["in", 0, 0]], "output_layers": [["out", 0, 0]],
        "layers": [
            {"class_name": "InputLayer", "name": "in", "config": {"name": "in", "batch_input_shape": [None, 6]}, "inbound_nodes": []},
            {"class_name": "Reshape", "name": "rs", "config": {"name": "rs", "target_shape": [3, 2]}, "inbound_nodes": [[["in", 0, 0, {}]]]},
            {"class_name": "Masking", "name": "mk", "config": {"name": "mk", "mask_value": 0.0}, "inbound_nodes": [[["rs", 0, 0, {}]]]},
            {"class_name": "SimpleRNN", "name": "rnn", "config": {"name": "rnn", "units": 2, "activation": "tanh", "return_sequences": False}, "inbound_nodes": [[["mk", 0, 0, {}]]]},
            {"class_name": "Dense", "name": "out", "config": {"name": "out", "units": 2, "activation": "linear"}, "inbound_nodes": [[["rnn", 0, 0, {}]]]},
        ]}}
    w = {"rnn": [arr(2, 2), arr(2, 2), arr(2)], "out": [arr(2, 2), arr(2)]}
    net = KerasModelImport.importKerasModelAndWeights(json.dumps(cfg), w)
    x = torch.randn(2, 6)
    x[1, 2:] = 0.0                                                      # example 1: one real step, two masked
    W, U, b = (t(a) for a in w["rnn"])
    ref = []
    for e, steps in ((0, 3), (1, 1)):
        h = torch.zeros(2)
        for s in range(steps):
            h = (x[e].reshape(3, 2)[s] @ W + h @ U + b).tanh()
        ref.append(h @ t(w["out"][0]) + t(w["out"][1]))
    assert torch.allclose(out(net, x), torch.stack(ref), atol=1e-5)


def test_attention_layer_becomes_the_dot_product_vertex():
    def model(causal, three):
        ins = [["q", 0, 0, {}], ["v", 0, 0, {}]] + ([["k", 0, 0, {}]] if three else [])
        names = ["q", "v"] + (["k"] if three else [])
        return json.dumps({"class_name": "Model", "config": {
            "name": "m", "input_layers": [[n, 0, 0] for n in names], "output_layers": [["att", 0, 0]],
            "layers": [{"class_name": "InputLayer", "name": n, "config": {"name": n, "batch_input_shape": [None, 4 if n == "q" else 5, 3]}, "inbound_nodes": []} for n in names] +
                      [{"class_name": "Attention", "name": "att", "config": {"name": "att", "use_scale": True, "causal": causal}, "inbound_nodes": [ins]}]}})
    q, v, k = torch.randn(2, 4, 3), torch.randn(2, 5, 3), torch.randn(2, 5, 3)
    cf = lambda a: a.permute(0, 2, 1).contiguous()
    for causal in (False, True):
        for three in (False, True):
            net = KerasModelImport.importKerasModelAndWeights(model(causal, three), {"att": [np.asarray(0.7, dtype="f4")]})
            kk = k if three else v
            s = 0.7 * q @ kk.transpose(1, 2)
            if causal:
                s = s.masked_fill(torch.ones(4, 5).triu(1) > 0, float("-inf"))
            ref = s.softmax(-1) @ v
            got = net.output(*([cf(q), cf(v)] + ([cf(k)] if three else [])))
            got = got[0] if isinstance(got, (list, tuple)) else got
            got = torch.as_tensor(np.asarray(got.numpy() if hasattr(got, "numpy") else got))
            assert torch.allclose(got.permute(0, 2, 1), ref, atol=1e-5), (causal, three)
    with pytest.raises(Exception, match="score mode"):
        KerasModelImport.importKerasModelAndWeights(model(False, False).replace('"use_scale": true', '"use_scale": true, "score_mode": "concat"'))
