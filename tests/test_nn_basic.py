"""MultiLayerNetwork / ComputationGraph basics: configuration JSON round trip, flat parameter layout, training
convergence, updater formulas against hand-written references, ModelSerializer zip round trip (bit-exact), layer
output shapes, tBPTT and rnnTimeStep.  Mirrors the intent of deeplearning4j-core's MultiLayerTest,
TestComputationGraphNetwork, TestUpdaters and ModelSerializerTest."""
import io
import math
import zipfile

import numpy as np
import pytest
import torch

from deeplearning4j_b200 import Nd4j, nn
from deeplearning4j_b200.data import DataSet


def _mlp_conf(updater=None, seed=12345):
    return (nn.NeuralNetConfiguration.Builder().seed(seed).updater(updater or nn.Adam(1e-2)).weightInit("XAVIER").list()
            .layer(nn.DenseLayer(nIn=4, nOut=16, activation="relu"))
            .layer(nn.DenseLayer(nIn=16, nOut=16, activation="tanh"))
            .layer(nn.OutputLayer("MCXENT", nIn=16, nOut=3, activation="softmax"))
            .build())


def _blobs(n=150, seed=0):
    rng = np.random.default_rng(seed)
    centers = np.array([[2, 0, 0, 0], [0, 2, 0, 0], [0, 0, 2, 0]], dtype=np.float32)
    lab = rng.integers(0, 3, size=n)
    x = centers[lab] + 0.3 * rng.normal(size=(n, 4)).astype(np.float32)
    return x.astype(np.float32), np.eye(3, dtype=np.float32)[lab]


def test_configuration_json_round_trip():
    conf = _mlp_conf()
    js = conf.toJson()
    back = nn.MultiLayerConfiguration.fromJson(js)
    assert back.toJson() == js
    assert "org.deeplearning4j.nn.conf.layers.DenseLayer" in js
    net = nn.MultiLayerNetwork(back)
    net.init()
    assert net.numParams() == 4 * 16 + 16 + 16 * 16 + 16 + 16 * 3 + 3


def test_flat_params_layout_and_views():
    net = nn.MultiLayerNetwork(_mlp_conf())
    net.init()
    flat = net.params()
    assert flat.length() == net.numParams()
    table = net.paramTable()
    assert list(table.keys())[:2] == ["0_W", "0_b"]
    w0 = table["0_W"]
    assert w0.shape() == (4, 16)
    # DL4J stores dense weights in 'f' order: the first nIn entries of the flat vector are column 0 of W
    np.testing.assert_array_equal(flat.numpy().ravel()[:4], w0.numpy()[:, 0])
    # views alias the flat buffer
    net.setParam("0_b", Nd4j.ones(1, 16))
    assert float(net.params().numpy().ravel()[64:80].sum()) == 16.0
    same = nn.MultiLayerNetwork(_mlp_conf())
    same.init()
    same.setParams(net.params())
    assert same.params().equals(net.params())


def test_same_seed_same_init_and_training_converges():
    a, b = nn.MultiLayerNetwork(_mlp_conf()), nn.MultiLayerNetwork(_mlp_conf())
    a.init()
    b.init()
    assert a.params().equals(b.params())
    x, y = _blobs()
    ds = DataSet(Nd4j.create(x), Nd4j.create(y))
    s0 = a.score(ds)
    for _ in range(60):
        a.fit(ds)
    assert a.score(ds) < 0.3 * s0
    ev = a.evaluate(__import__("deeplearning4j_b200.data", fromlist=["ListDataSetIterator"]).ListDataSetIterator([ds], 150))
    assert ev.accuracy() > 0.95
    out = a.output(Nd4j.create(x[:5]))
    np.testing.assert_allclose(out.numpy().sum(1), np.ones(5), rtol=1e-5)
    assert a.predict(Nd4j.create(x[:5])) == list(np.argmax(out.numpy(), 1))


def _one_step(updater, grad, steps=3):
    """Run ``steps`` updates of a single scalar-free parameter vector through the framework's updater."""
    conf = (nn.NeuralNetConfiguration.Builder().seed(1).updater(updater).list()
            .layer(nn.DenseLayer(nIn=2, nOut=2, hasBias=False, activation="identity"))
            .layer(nn.LossLayer("MSE", activation="identity")).build())
    net = nn.MultiLayerNetwork(conf)
    net.init()
    p0 = net.params().numpy().ravel().copy()
    hist = [p0]
    for i in range(steps):
        net.flat_grads.copy_(torch.as_tensor(grad))
        net._ensure_updater().update(i, 0)
        hist.append(net.params().numpy().ravel().copy())
    return hist


def test_updater_formulas():
    g = np.array([0.5, -1.0, 2.0, 0.25], dtype=np.float32)
    # SGD
    h = _one_step(nn.Sgd(0.1), g, 2)
    np.testing.assert_allclose(h[1], h[0] - 0.1 * g, rtol=1e-6)
    # Nesterovs (DL4J form): v' = mu v - lr g ; update = mu v - (1 + mu) v'  => p += -mu v + (1 + mu) v'
    mu, lr = 0.9, 0.1
    h = _one_step(nn.Nesterovs(lr, mu), g, 3)
    v = np.zeros(4, dtype=np.float32)
    p = h[0].copy()
    for k in range(3):
        v_prev = v
        v = mu * v - lr * g
        p = p - (mu * v_prev - (1 + mu) * v)
        np.testing.assert_allclose(h[k + 1], p, rtol=1e-5, atol=1e-6)
    # Adam
    lr, b1, b2, eps = 0.01, 0.9, 0.999, 1e-8
    h = _one_step(nn.Adam(lr), g, 3)
    m, v2, p = np.zeros(4), np.zeros(4), h[0].astype(np.float64)
    for k in range(3):
        t = k + 1
        m = b1 * m + (1 - b1) * g
        v2 = b2 * v2 + (1 - b2) * g * g
        alpha = lr * math.sqrt(1 - b2 ** t) / (1 - b1 ** t)
        p = p - alpha * m / (np.sqrt(v2) + eps)
        np.testing.assert_allclose(h[k + 1], p, rtol=1e-5, atol=1e-7)
    # RmsProp: cache = d cache + (1 - d) g^2 ; p -= lr g / sqrt(cache + eps)
    lr, d, eps = 0.1, 0.95, 1e-8
    h = _one_step(nn.RmsProp(lr), g, 2)
    cache, p = np.full(4, eps), h[0].astype(np.float64)
    for k in range(2):
        cache = d * cache + (1 - d) * g * g
        p = p - lr * g / np.sqrt(cache + eps)
        np.testing.assert_allclose(h[k + 1], p, rtol=1e-4, atol=1e-6)
    # AdaGrad
    lr, eps = 0.1, 1e-6
    h = _one_step(nn.AdaGrad(lr), g, 2)
    acc, p = np.full(4, eps), h[0].astype(np.float64)
    for k in range(2):
        acc = acc + g * g
        p = p - lr * g / (np.sqrt(acc) + eps)
        np.testing.assert_allclose(h[k + 1], p, rtol=1e-4, atol=1e-6)


def test_l2_and_weight_decay_change_the_update():
    x, y = _blobs(32)
    ds = DataSet(Nd4j.create(x), Nd4j.create(y))

    def run(**kw):
        b = nn.NeuralNetConfiguration.Builder().seed(7).updater(nn.Sgd(0.1))
        for k, v in kw.items():
            getattr(b, k)(v)
        conf = (b.list().layer(nn.DenseLayer(nIn=4, nOut=3, activation="identity"))
                .layer(nn.OutputLayer("MCXENT", nIn=3, nOut=3, activation="softmax")).build())
        net = nn.MultiLayerNetwork(conf)
        net.init()
        p0 = net.params().numpy().copy()
        net.fit(ds)
        return p0, net.params().numpy().copy(), net
    p0, plain, _ = run()
    _, l2, net = run(l2=0.1)
    w_idx = slice(0, 12)
    # L2 adds coeff * w to the weight gradient (not to biases): difference = -lr * l2 * w
    np.testing.assert_allclose((l2 - plain).ravel()[w_idx], (-0.1 * 0.1 * p0).ravel()[w_idx], rtol=1e-3, atol=1e-6)
    np.testing.assert_allclose((l2 - plain).ravel()[12:15], 0.0, atol=1e-7)
    assert net.score() > 0


def test_model_serializer_zip_round_trip_is_bit_exact(tmp_path):
    net = nn.MultiLayerNetwork(_mlp_conf())
    net.init()
    x, y = _blobs(40)
    ds = DataSet(Nd4j.create(x), Nd4j.create(y))
    for _ in range(3):
        net.fit(ds)
    path = str(tmp_path / "model.zip")
    nn.ModelSerializer.writeModel(net, path, True)
    with zipfile.ZipFile(path) as z:
        names = set(z.namelist())
    assert {"configuration.json", "coefficients.bin", "updaterState.bin"} <= names
    back = nn.ModelSerializer.restoreMultiLayerNetwork(path, True)
    assert np.array_equal(back.params().numpy(), net.params().numpy())
    assert np.array_equal(back.getUpdater().getStateViewArray().numpy(), net.getUpdater().getStateViewArray().numpy())
    np.testing.assert_array_equal(back.output(Nd4j.create(x)).numpy(), net.output(Nd4j.create(x)).numpy())
    # training continues identically from the restored updater state
    net.fit(ds)
    back.fit(ds)
    assert np.array_equal(back.params().numpy(), net.params().numpy())
    assert nn.ModelGuesser.loadModelGuess(path).numParams() == net.numParams()


def test_computation_graph_merge_and_elementwise():
    conf = (nn.NeuralNetConfiguration.Builder().seed(3).updater(nn.Adam(1e-2)).graphBuilder()
            .addInputs("a", "b")
            .addLayer("da", nn.DenseLayer(nIn=4, nOut=8, activation="relu"), "a")
            .addLayer("db", nn.DenseLayer(nIn=4, nOut=8, activation="relu"), "b")
            .addVertex("sum", nn.ElementWiseVertex("Add"), "da", "db")
            .addVertex("cat", nn.MergeVertex(), "sum", "da")
            .addLayer("out", nn.OutputLayer("MCXENT", nIn=16, nOut=3, activation="softmax"), "cat")
            .setOutputs("out").build())
    js = conf.toJson()
    assert nn.ComputationGraphConfiguration.fromJson(js).toJson() == js
    g = nn.ComputationGraph(conf)
    g.init()
    x, y = _blobs(60)
    xa, xb, lab = Nd4j.create(x), Nd4j.create(x[::-1].copy()), Nd4j.create(y)
    out = g.output(xa, xb)[0]
    assert out.shape() == (60, 3)
    from deeplearning4j_b200.data import MultiDataSet
    mds = MultiDataSet([xa, xb], [lab])
    s0 = g.score(mds)
    for _ in range(40):
        g.fit(mds)
    assert g.score(mds) < 0.5 * s0
    acts = g.feedForward([xa, xb], False)
    assert set(acts) >= {"da", "db", "sum", "cat", "out"} and acts["cat"].shape() == (60, 16)


def test_cnn_shapes_and_preprocessors():
    conf = (nn.NeuralNetConfiguration.Builder().seed(1).updater(nn.Sgd(0.01)).list()
            .layer(nn.ConvolutionLayer(kernelSize=(3, 3), stride=(1, 1), nOut=4, activation="relu"))
            .layer(nn.SubsamplingLayer(poolingType="MAX", kernelSize=(2, 2), stride=(2, 2)))
            .layer(nn.BatchNormalization())
            .layer(nn.DenseLayer(nOut=10, activation="relu"))
            .layer(nn.OutputLayer("MCXENT", nOut=3, activation="softmax"))
            .setInputType(nn.InputType.convolutional(8, 8, 1)).build())
    net = nn.MultiLayerNetwork(conf)
    net.init()
    x = Nd4j.rand(5, 1, 8, 8)
    acts = net.feedForward(x, False)
    assert acts[1].shape() == (5, 4, 6, 6) and acts[2].shape() == (5, 4, 3, 3) and acts[-1].shape() == (5, 3)
    # nIn inferred from the input type: 4 * 3 * 3 features into the dense layer
    assert net.getLayer(3).nIn == 36
    y = Nd4j.create(np.eye(3, dtype=np.float32)[[0, 1, 2, 0, 1]])
    net.fit(DataSet(x, y))
    assert math.isfinite(net.score())


def test_tbptt_and_rnn_time_step_match_full_forward():
    conf = (nn.NeuralNetConfiguration.Builder().seed(5).updater(nn.Adam(1e-2)).list()
            .layer(nn.LSTM(nIn=3, nOut=6, activation="tanh"))
            .layer(nn.RnnOutputLayer("MCXENT", nIn=6, nOut=2, activation="softmax"))
            .backpropType("TruncatedBPTT").tBPTTForwardLength(4).tBPTTBackwardLength(4).build())
    net = nn.MultiLayerNetwork(conf)
    net.init()
    rng = np.random.default_rng(0)
    x = rng.normal(size=(2, 3, 12)).astype(np.float32)
    lab = np.zeros((2, 2, 12), dtype=np.float32)
    lab[:, 0, ::2] = 1
    lab[:, 1, 1::2] = 1
    full = net.output(Nd4j.create(x)).numpy()
    net.rnnClearPreviousState()
    steps = [net.rnnTimeStep(Nd4j.create(x[:, :, t:t + 1])).numpy() for t in range(12)]
    np.testing.assert_allclose(np.concatenate(steps, 2), full, rtol=1e-4, atol=1e-5)
    net.rnnClearPreviousState()
    s0 = net.score(DataSet(Nd4j.create(x), Nd4j.create(lab)))
    for _ in range(30):
        net.fit(DataSet(Nd4j.create(x), Nd4j.create(lab)))
    assert net.score(DataSet(Nd4j.create(x), Nd4j.create(lab))) < s0
    assert net.getIterationCount() == 30 * 3          # 12 steps / tBPTT length 4 = 3 parameter updates per fit


def test_gradient_and_score_api():
    net = nn.MultiLayerNetwork(_mlp_conf(nn.Sgd(0.1)))
    net.init()
    x, y = _blobs(16)
    net.setInput(Nd4j.create(x))
    net.setLabels(Nd4j.create(y))
    net.computeGradientAndScore()
    g = net.gradient()
    assert g.gradient().length() == net.numParams()
    assert set(g.gradientForVariable().keys()) == set(net.paramTable().keys())
    assert math.isfinite(net.score()) and net.score() > 0


def test_graph_fuses_batchnorm_add_relu_chains_without_changing_results():
    def build():
        return (nn.NeuralNetConfiguration.Builder().seed(9).updater(nn.Sgd(0.05)).graphBuilder()
                .addInputs("in")
                .addLayer("c1", nn.ConvolutionLayer(kernelSize=(3, 3), padding=(1, 1), nIn=8, nOut=8, activation="identity"), "in")
                .addLayer("bn1", nn.BatchNormalization(nOut=8), "c1")
                .addLayer("r1", nn.ActivationLayer("relu"), "bn1")
                .addLayer("c2", nn.ConvolutionLayer(kernelSize=(1, 1), nIn=8, nOut=8, activation="identity"), "r1")
                .addLayer("bn2", nn.BatchNormalization(nOut=8), "c2")
                .addVertex("add", nn.ElementWiseVertex("Add"), "bn2", "in")
                .addLayer("r2", nn.ActivationLayer("relu"), "add")
                .addLayer("gp", nn.GlobalPoolingLayer("AVG"), "r2")
                .addLayer("out", nn.OutputLayer("MCXENT", nIn=8, nOut=3, activation="softmax"), "gp")
                .setOutputs("out").setInputTypes(nn.InputType.convolutional(6, 6, 8)).build())
    a, b = nn.ComputationGraph(build()), nn.ComputationGraph(build())
    a.init()
    b.init()
    plan = a._fusion_plan()
    assert plan["bn1"] == ("bn_relu",) and plan["r1"] == ("alias", "bn1")
    assert plan["bn2"] == ("defer",) and plan["add"] == ("bn_add_relu", "bn2", "in") and plan["r2"] == ("alias", "add")
    b._fuse_plan = {}                                  # reference: no fusion
    rng = np.random.default_rng(1)
    x = Nd4j.create(rng.normal(size=(4, 8, 6, 6)).astype(np.float32))
    y = Nd4j.create(np.eye(3, dtype=np.float32)[[0, 1, 2, 1]])
    from deeplearning4j_b200.data import DataSet as DS
    for _ in range(3):
        a.fit(DS(x, y))
        b.fit(DS(x, y))
    np.testing.assert_allclose(a.params().numpy(), b.params().numpy(), rtol=1e-5, atol=1e-6)
    # feedForward still exposes every intermediate activation (fusion is only used on the loss path)
    acts = a.feedForward([x], False)
    assert float(acts["bn1"].numpy().min()) < 0 <= float(acts["r1"].numpy().min())
