"""Declarable-op registry: every reference op name resolves, and a broad sample of ops from each family matches a
numpy / torch oracle.  Mirrors the intent of libnd4j's DeclarableOpsTests* and nd4j's OpValidation suites."""
import numpy as np
import pytest
import torch

import deeplearning4j_b200.samediff  # noqa: F401  (registers the graph-only ops)
from deeplearning4j_b200.ops import registry

RNG = np.random.default_rng(42)
X = RNG.normal(size=(3, 4)).astype(np.float32)
Y = RNG.normal(size=(3, 4)).astype(np.float32)
P = np.abs(X) + 0.5


def run(name, *ins, **kw):
    r = registry.execute(name, [torch.as_tensor(i) if isinstance(i, np.ndarray) else i for i in ins], **kw)
    if isinstance(r, (tuple, list)):
        return [t.numpy() if isinstance(t, torch.Tensor) else t for t in r]
    return r.numpy() if isinstance(r, torch.Tensor) else r


def test_registry_size_hashes_and_lookup():
    names = registry.names()
    assert len(names) >= 500
    for n in ("conv2d", "lstmLayer", "softmax_cross_entropy_loss", "matmul", "layer_norm", "encode_threshold", "adam_updater"):
        assert registry.has(n), n
    # op hashes are stable 64-bit ids usable as FlatBuffers op numbers and they round-trip to names
    h = registry.op_hash("conv2d")
    assert isinstance(h, int) and registry.name_for_hash(h) == "conv2d"
    assert registry.op_hash("conv2d") != registry.op_hash("conv3dnew")
    with pytest.raises(Exception):
        registry.get("definitely_not_an_op")


UNARY = {
    "abs": np.abs, "neg": np.negative, "exp": np.exp, "tanh": np.tanh, "sin": np.sin, "cos": np.cos, "floor": np.floor,
    "ceil": np.ceil, "sign": np.sign, "square": np.square, "cube": lambda x: x ** 3, "sigmoid": lambda x: 1 / (1 + np.exp(-x)),
    "relu": lambda x: np.maximum(x, 0), "relu6": lambda x: np.clip(x, 0, 6), "softplus": lambda x: np.log1p(np.exp(x)),
    "softsign": lambda x: x / (1 + np.abs(x)), "expm1": np.expm1, "erf": lambda x: torch.erf(torch.as_tensor(x)).numpy(),
    "atan": np.arctan, "sinh": np.sinh, "cosh": np.cosh, "asinh": np.arcsinh, "hardtanh": lambda x: np.clip(x, -1, 1),
    "swish": lambda x: x / (1 + np.exp(-x)), "round": np.rint, "rint": np.rint, "identity": lambda x: x,
    "hardsigmoid": lambda x: np.clip(0.2 * x + 0.5, 0, 1), "elu": lambda x: np.where(x > 0, x, np.exp(x) - 1),
    "mish": lambda x: x * np.tanh(np.log1p(np.exp(x))), "gelu": lambda x: x / (1 + np.exp(-1.702 * x)),
}
UNARY_POS = {"log": np.log, "sqrt": np.sqrt, "rsqrt": lambda x: 1 / np.sqrt(x), "log1p": np.log1p, "reciprocal": lambda x: 1 / x,
             "log2": np.log2, "log10": np.log10}


@pytest.mark.parametrize("name", sorted(UNARY))
def test_unary_elementwise(name):
    np.testing.assert_allclose(run(name, X), UNARY[name](X), rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("name", sorted(UNARY_POS))
def test_unary_positive_domain(name):
    np.testing.assert_allclose(run(name, P), UNARY_POS[name](P), rtol=2e-5, atol=2e-6)


BINARY = {
    "add": np.add, "subtract": np.subtract, "multiply": np.multiply, "divide": np.divide, "maximum": np.maximum,
    "minimum": np.minimum, "squaredsubtract": lambda a, b: (a - b) ** 2, "reversesubtract": lambda a, b: b - a,
    "reversedivide": lambda a, b: b / a, "atan2": np.arctan2, "floormod": lambda a, b: a - np.floor(a / b) * b,
    "greater": np.greater, "less": np.less, "greater_equal": np.greater_equal, "less_equal": np.less_equal,
    "equals": np.equal, "not_equals": np.not_equal,
}


@pytest.mark.parametrize("name", sorted(BINARY))
def test_binary_broadcastable(name):
    got = run(name, X, Y)
    np.testing.assert_allclose(got.astype(np.float32), BINARY[name](X, Y).astype(np.float32), rtol=2e-5, atol=2e-6)
    # broadcasting a row vector
    got = run(name, X, Y[0])
    np.testing.assert_allclose(got.astype(np.float32), BINARY[name](X, Y[0]).astype(np.float32), rtol=2e-5, atol=2e-6)


REDUCE = {
    "reduce_sum": np.sum, "reduce_mean": np.mean, "reduce_max": np.max, "reduce_min": np.min, "reduce_prod": np.prod,
    "reduce_norm1": lambda x, axis, keepdims: np.abs(x).sum(axis=axis, keepdims=keepdims),
    "reduce_norm2": lambda x, axis, keepdims: np.sqrt((x * x).sum(axis=axis, keepdims=keepdims)),
    "reduce_sqnorm": lambda x, axis, keepdims: (x * x).sum(axis=axis, keepdims=keepdims),
    "reduce_norm_max": lambda x, axis, keepdims: np.abs(x).max(axis=axis, keepdims=keepdims),
    "reduce_logsumexp": lambda x, axis, keepdims: np.log(np.exp(x).sum(axis=axis, keepdims=keepdims)),
    "reduce_variance": np.var, "reduce_stdev": np.std,
}


@pytest.mark.parametrize("name", sorted(REDUCE))
@pytest.mark.parametrize("dims,keep", [((1,), False), ((0,), True), (None, False)])
def test_reductions(name, dims, keep):
    kw = {"keepDims": keep}
    if dims is not None:
        kw["dimensions"] = list(dims)
    ref = REDUCE[name](X, axis=dims, keepdims=keep)
    np.testing.assert_allclose(run(name, X, **kw), ref, rtol=2e-5, atol=2e-6)


def test_index_reductions_and_cumulative():
    assert run("argmax", X, dimensions=[1]).tolist() == X.argmax(1).tolist()
    assert run("argmin", X, dimensions=[0]).tolist() == X.argmin(0).tolist()
    np.testing.assert_allclose(run("cumsum", X, dimensions=[1]), X.cumsum(1), rtol=1e-5)
    np.testing.assert_allclose(run("cumsum", X, dimensions=[1], exclusive=True), X.cumsum(1) - X, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(run("cumsum", X, dimensions=[1], reverse=True), X[:, ::-1].cumsum(1)[:, ::-1], rtol=1e-5)
    np.testing.assert_allclose(run("cumprod", P, dimensions=[0]), P.cumprod(0), rtol=1e-5)
    v, i = run("top_k", X, k=2)
    np.testing.assert_allclose(v, -np.sort(-X, 1)[:, :2])
    assert run("in_top_k", X, X.argmax(1), k=1).all()


def test_shape_ops():
    np.testing.assert_array_equal(run("reshape", X, shape=[4, 3]), X.reshape(4, 3))
    np.testing.assert_array_equal(run("permute", X, dimensions=[1, 0]), X.T)
    np.testing.assert_array_equal(run("transpose", X), X.T)
    np.testing.assert_array_equal(run("concat", X, Y, concatDimension=1), np.concatenate([X, Y], 1))
    np.testing.assert_array_equal(run("stack", X, Y, dimension=0), np.stack([X, Y]))
    parts = run("unstack", X, dimension=0)
    assert len(parts) == 3 and np.array_equal(parts[1], X[1])
    halves = run("split", X, numSplit=2, dimension=1)
    assert np.array_equal(halves[0], X[:, :2]) and np.array_equal(halves[1], X[:, 2:])
    np.testing.assert_array_equal(run("tile", X, reps=[2, 1]), np.tile(X, (2, 1)))
    np.testing.assert_array_equal(run("reverse", X, dimensions=[1]), X[:, ::-1])
    np.testing.assert_array_equal(run("slice", X, begin=[1, 1], size=[2, 2]), X[1:3, 1:3])
    np.testing.assert_array_equal(run("strided_slice", X, begin=[0, 0], end=[3, 4], strides=[2, 2]), X[::2, ::2])
    np.testing.assert_array_equal(run("gather", X, np.array([2, 0]), axis=0), X[[2, 0]])
    np.testing.assert_array_equal(run("expand_dims", X, axis=1).shape, (3, 1, 4))
    np.testing.assert_array_equal(run("squeeze", X[:, None], dimensions=[1]), X)
    np.testing.assert_array_equal(run("pad", X, np.array([[1, 1], [0, 2]]), mode=0, padValue=7.0),
                                  np.pad(X, ((1, 1), (0, 2)), constant_values=7.0))
    np.testing.assert_array_equal(run("onehot", np.array([0, 2, 1]), depth=3), np.eye(3, dtype=np.float32)[[0, 2, 1]])
    np.testing.assert_array_equal(run("diag", np.array([1.0, 2.0], dtype=np.float32)), np.diag([1.0, 2.0]).astype(np.float32))
    np.testing.assert_array_equal(run("diag_part", np.arange(9, dtype=np.float32).reshape(3, 3)), [0, 4, 8])
    assert run("shape_of", X).tolist() == [3, 4] and int(run("rank", X)) == 2 and int(run("size", X)) == 12
    np.testing.assert_array_equal(run("where", X > 0, X, Y), np.where(X > 0, X, Y))
    np.testing.assert_array_equal(run("clipbyvalue", X, clipValueMin=-0.5, clipValueMax=0.5), np.clip(X, -0.5, 0.5))
    np.testing.assert_array_equal(run("space_to_depth", np.arange(16, dtype=np.float32).reshape(1, 1, 4, 4), blockSize=2).shape, (1, 4, 2, 2))
    s2d = run("space_to_depth", np.arange(16, dtype=np.float32).reshape(1, 1, 4, 4), blockSize=2)
    np.testing.assert_array_equal(run("depth_to_space", s2d, blockSize=2), np.arange(16, dtype=np.float32).reshape(1, 1, 4, 4))


def test_scatter_segment_and_partition_ops():
    base = np.zeros((4, 2), dtype=np.float32)
    upd = np.ones((3, 2), dtype=np.float32)
    idx = np.array([0, 2, 0])
    got = run("scatter_add", base, idx, upd)
    np.testing.assert_array_equal(got, [[2, 2], [0, 0], [1, 1], [0, 0]])
    got = run("scatter_upd", base, np.array([1, 3]), upd[:2] * 5)
    np.testing.assert_array_equal(got, [[0, 0], [5, 5], [0, 0], [5, 5]])
    data = np.array([1.0, 2.0, 3.0, 4.0, 5.0], dtype=np.float32)
    ids = np.array([0, 0, 1, 2, 2])
    np.testing.assert_array_equal(run("segment_sum", data, ids), [3, 3, 9])
    np.testing.assert_array_equal(run("segment_max", data, ids), [2, 3, 5])
    np.testing.assert_array_equal(run("unsorted_segment_sum", data, np.array([2, 0, 2, 1, 0]), numSegments=3), [7, 4, 4])
    parts = run("dynamic_partition", data, np.array([0, 1, 0, 1, 0]), numPartitions=2)
    assert parts[0].tolist() == [1, 3, 5] and parts[1].tolist() == [2, 4]
    np.testing.assert_array_equal(run("sequence_mask", np.array([1, 3]), maxLen=4).astype(int), [[1, 0, 0, 0], [1, 1, 1, 0]])
    cm = run("confusion_matrix", np.array([0, 1, 1]), np.array([0, 1, 0]), numClasses=2)
    np.testing.assert_array_equal(cm, [[1, 0], [1, 1]])
    u = run("unique", np.array([3, 1, 3, 2, 1]))
    assert sorted(u[0].tolist()) == [1, 2, 3]


def test_linalg_ops():
    a = RNG.normal(size=(4, 4)).astype(np.float64)
    spd = a @ a.T + 4 * np.eye(4)
    np.testing.assert_allclose(run("matmul", X, Y, transposeY=True), X @ Y.T, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(run("matrix_inverse", spd) @ spd, np.eye(4), atol=1e-8)
    np.testing.assert_allclose(run("matrix_determinant", spd), np.linalg.det(spd), rtol=1e-8)
    L = run("cholesky", spd)
    np.testing.assert_allclose(L @ L.T, spd, rtol=1e-8)
    q, r = run("qr", a)
    np.testing.assert_allclose(q @ r, a, atol=1e-8)
    s = run("svd", a, computeUv=False)
    s = s[0] if isinstance(s, list) else s
    np.testing.assert_allclose(np.sort(s)[::-1], np.linalg.svd(a, compute_uv=False), rtol=1e-8)
    np.testing.assert_allclose(run("trace", spd), np.trace(spd))
    np.testing.assert_allclose(run("cross", X[:, :3], Y[:, :3]), np.cross(X[:, :3], Y[:, :3]), rtol=1e-5, atol=1e-6)
    b = RNG.normal(size=(4, 2))
    np.testing.assert_allclose(run("solve", spd, b), np.linalg.solve(spd, b), rtol=1e-8)
    np.testing.assert_allclose(run("tensormmul", X, Y.T.copy(), dimensionsX=[1], dimensionsY=[0]), X @ Y.T, rtol=1e-5, atol=1e-5)


def test_nn_ops_against_torch():
    t = torch.as_tensor
    np.testing.assert_allclose(run("softmax", X, dimension=1), torch.softmax(t(X), 1).numpy(), rtol=1e-6)
    np.testing.assert_allclose(run("log_softmax", X, dimension=1), torch.log_softmax(t(X), 1).numpy(), rtol=1e-5, atol=1e-6)
    g, b = np.ones(4, dtype=np.float32) * 1.5, np.ones(4, dtype=np.float32) * 0.1
    np.testing.assert_allclose(run("layer_norm", X, g, b), torch.nn.functional.layer_norm(t(X), (4,), t(g), t(b)).numpy(), rtol=1e-4, atol=1e-5)
    img = RNG.normal(size=(2, 3, 8, 8)).astype(np.float32)
    w = RNG.normal(size=(5, 3, 3, 3)).astype(np.float32)
    bias = RNG.normal(size=(5,)).astype(np.float32)
    ref = torch.nn.functional.conv2d(t(img), t(w), t(bias), stride=1, padding=1).numpy()
    np.testing.assert_allclose(run("conv2d", img, w, bias, kH=3, kW=3, pH=1, pW=1, wFormat=1), ref, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(run("maxpool2d", img, kH=2, kW=2, sH=2, sW=2), torch.nn.functional.max_pool2d(t(img), 2).numpy())
    np.testing.assert_allclose(run("avgpool2d", img, kH=2, kW=2, sH=2, sW=2), torch.nn.functional.avg_pool2d(t(img), 2).numpy(), rtol=1e-6)
    m, v = img.mean((0, 2, 3)), img.var((0, 2, 3))
    ref = torch.nn.functional.batch_norm(t(img), t(m), t(v), None, None, False, 0.0, 1e-5).numpy()
    np.testing.assert_allclose(run("batchnorm", img, m, v, epsilon=1e-5, axis=(1,)), ref, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(run("upsampling2d", img, scaleH=2, scaleW=2), np.repeat(np.repeat(img, 2, 2), 2, 3))
    np.testing.assert_allclose(run("leakyrelu", X, alpha=0.1), np.where(X > 0, X, 0.1 * X), rtol=1e-6)
    np.testing.assert_allclose(run("standardize", X, dimensions=[1]).mean(1), 0, atol=1e-6)
    d = run("dropout", np.ones((100, 100), dtype=np.float32), probValue=0.5, seed=3, training=True)
    assert 0.4 < (d == 0).mean() < 0.6 and abs(d.mean() - 1.0) < 0.1


def test_loss_ops():
    logits = RNG.normal(size=(5, 3)).astype(np.float32)
    lab_idx = np.array([0, 2, 1, 1, 0])
    onehot = np.eye(3, dtype=np.float32)[lab_idx]
    ref = torch.nn.functional.cross_entropy(torch.as_tensor(logits), torch.as_tensor(lab_idx)).item()
    w = np.ones((1,), dtype=np.float32)
    assert abs(float(run("softmax_cross_entropy_loss", logits, w, onehot, reductionMode=3)) - ref) < 1e-5
    assert abs(float(np.mean(run("sparse_softmax_cross_entropy_loss_with_logits", lab_idx, logits))) - ref) < 1e-5
    pred = RNG.normal(size=(5, 3)).astype(np.float32)
    assert abs(float(run("mean_sqerr_loss", pred, w, onehot, reductionMode=3)) - float(((pred - onehot) ** 2).mean())) < 1e-5
    assert abs(float(run("absolute_difference_loss", pred, w, onehot, reductionMode=3)) - float(np.abs(pred - onehot).mean())) < 1e-5
    ref = torch.nn.functional.binary_cross_entropy_with_logits(torch.as_tensor(pred), torch.as_tensor(onehot)).item()
    assert abs(float(run("sigm_cross_entropy_loss", pred, w, onehot, reductionMode=3)) - ref) < 1e-5
    ref = torch.nn.functional.huber_loss(torch.as_tensor(pred), torch.as_tensor(onehot), delta=1.0).item()
    assert abs(float(run("huber_loss", pred, w, onehot, reductionMode=3, delta=1.0)) - ref) < 1e-5


def test_random_ops_are_seeded_and_distributed():
    registry.execute("set_seed", [], seed=11)
    a = run("random_normal", [2000], mean=1.0, stdev=2.0)
    registry.execute("set_seed", [], seed=11)
    b = run("random_normal", [2000], mean=1.0, stdev=2.0)
    assert np.array_equal(a, b) and abs(a.mean() - 1.0) < 0.2 and abs(a.std() - 2.0) < 0.2
    u = run("randomuniform", [2000], min=-1.0, max=3.0)
    assert u.min() >= -1.0 and u.max() <= 3.0 and abs(u.mean() - 1.0) < 0.2
    be = run("random_bernoulli", [4000], p=0.25)
    assert abs(be.mean() - 0.25) < 0.05


def test_image_ops():
    img = RNG.uniform(size=(1, 4, 4, 3)).astype(np.float32)
    up = run("resize_nearest_neighbor", img, height=8, width=8)
    assert up.shape == (1, 8, 8, 3) and np.array_equal(up[0, ::2, ::2], img[0])
    bl = run("resize_bilinear", img, height=8, width=8)
    assert bl.shape == (1, 8, 8, 3) and bl.min() >= img.min() - 1e-6 and bl.max() <= img.max() + 1e-6
    hsv = run("rgb_to_hsv", img)
    np.testing.assert_allclose(run("hsv_to_rgb", hsv), img, atol=1e-5)
    boxes = np.array([[0, 0, 1, 1], [0, 0, 0.9, 0.9], [0.5, 0.5, 1, 1]], dtype=np.float32)
    keep = run("non_max_suppression", boxes, np.array([0.9, 0.8, 0.7], dtype=np.float32), maxOutputSize=3, iouThreshold=0.5)
    assert keep.tolist() == [0, 2]


def test_updater_and_compression_ops():
    p = np.array([1.0, -2.0, 3.0], dtype=np.float32)
    g = np.array([0.1, 0.2, -0.3], dtype=np.float32)
    upd = run("sgd_updater", g, lr=0.5)
    upd = upd[0] if isinstance(upd, list) else upd
    np.testing.assert_allclose(upd, 0.5 * g, rtol=1e-6)
    x = np.array([0.0, 0.002, -0.0015, 0.0001, 0.003], dtype=np.float32)
    xt = torch.as_tensor(x.copy())
    enc_out = registry.execute("encode_threshold", [xt], threshold=1e-3)
    enc = enc_out[-1]
    residual = enc_out[0].numpy()
    np.testing.assert_allclose(residual, [0, 1e-3, -0.5e-3, 1e-4, 2e-3], atol=1e-7)        # what was sent is subtracted in place
    decoded = registry.execute("decode_threshold", [torch.zeros(5), enc])
    np.testing.assert_allclose(decoded.numpy(), [0, 1e-3, -1e-3, 0, 1e-3], atol=1e-9)
