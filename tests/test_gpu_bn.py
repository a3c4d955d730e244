"""Fused channels-last batch norm (+ residual) (+ ReLU) kernels against a plain PyTorch fp32 reference, and the
ResNet-style graph fusion on the GPU."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nat():
    from deeplearning4j_b200.ops import native
    native.require()
    assert native.available(), native.load_error()
    yield native
    native.check_status()


def _rel(a, b):
    """Worst element-wise error in units of (|reference element| + rms of the reference): ``_rel(a, b) < t`` is
    ``allclose(a, b, rtol=t, atol=t * rms(b))`` -- a region of small values that is wrong fails, which a max-norm ratio would hide."""
    a, b = a.detach().float(), b.detach().float()
    rms = float(b.pow(2).mean().sqrt()) + 1e-12
    return float(((a - b).abs() / (b.abs() + rms)).max())


def _ref(x, res, gamma, beta, eps, relu):
    xf = x.float()
    mean = xf.mean((0, 2, 3), keepdim=True)
    var = xf.var((0, 2, 3), unbiased=False, keepdim=True)
    y = (xf - mean) * torch.rsqrt(var + eps) * gamma.view(1, -1, 1, 1) + beta.view(1, -1, 1, 1)
    if res is not None:
        y = y + res.float()
    return (torch.relu(y) if relu else y), mean.flatten(), var.flatten()


@pytest.mark.parametrize("shape", [(8, 64, 14, 14), (3, 256, 7, 5), (16, 8, 9, 9), (2, 2048, 4, 4)])
@pytest.mark.parametrize("relu,with_res", [(False, False), (True, False), (True, True)])
def test_bn_act_train_forward_backward(nat, shape, relu, with_res):
    g = torch.Generator(device="cuda").manual_seed(sum(shape) + relu * 2 + with_res)
    N, C, H, W = shape
    x = (torch.randn(shape, device="cuda", generator=g) * 1.5 + 0.3).bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_(True)
    res = torch.randn(shape, device="cuda", generator=g).bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_(True) if with_res else None
    gamma = (torch.rand(C, device="cuda", generator=g) + 0.5).requires_grad_(True)
    beta = (torch.randn(C, device="cuda", generator=g) * 0.2).requires_grad_(True)
    run_mean = torch.zeros(C, device="cuda")
    run_sv = torch.zeros(C, device="cuda")              # log10(stdev) of a unit-variance start
    decay, eps = 0.9, 1e-5
    y = nat.bn_act_train(x, res, gamma, beta, run_mean, run_sv, True, decay, eps, relu)
    w = torch.randn(shape, device="cuda", generator=g)
    (y.float() * w).sum().backward()
    torch.cuda.synchronize()
    got = [x.grad.clone(), gamma.grad.clone(), beta.grad.clone()] + ([res.grad.clone()] if with_res else [])
    for t in (x, gamma, beta) + ((res,) if with_res else ()):
        t.grad = None
    ref, mean, var = _ref(x, res, gamma, beta, eps, relu)
    assert y.is_contiguous(memory_format=torch.channels_last)
    assert _rel(y, ref) < 2e-2
    (ref * w).sum().backward()
    want = [x.grad, gamma.grad, beta.grad] + ([res.grad] if with_res else [])
    for name, a, b in zip(("dx", "dgamma", "dbeta", "dres"), got, want):
        assert _rel(a, b) < 4e-2, (name, _rel(a, b))
    # running statistics: global = decay * global + (1 - decay) * batch, variance kept as log10(stdev)
    assert _rel(run_mean, (1 - decay) * mean.detach()) < 1e-2
    want_sv = 0.5 * torch.log10(decay * 1.0 + (1 - decay) * var.detach())
    assert float((run_sv - want_sv).abs().max()) < 5e-3


def test_bn_eval_and_add_relu(nat):
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(4, 128, 6, 6, device="cuda", generator=g).bfloat16().contiguous(memory_format=torch.channels_last)
    r = torch.randn(4, 128, 6, 6, device="cuda", generator=g).bfloat16().contiguous(memory_format=torch.channels_last)
    scale = torch.rand(128, device="cuda", generator=g) + 0.5
    shift = torch.randn(128, device="cuda", generator=g)
    y = nat.bn_act_eval(x, r, scale, shift, True)
    ref = torch.relu(x.float() * scale.view(1, -1, 1, 1) + shift.view(1, -1, 1, 1) + r.float())
    assert _rel(y, ref) < 1e-2
    a = x.clone().requires_grad_(True)
    b = r.clone().requires_grad_(True)
    z = nat.add_relu(a, b)
    z.float().sum().backward()
    zr = torch.relu(x.float() + r.float())
    assert _rel(z, zr) < 1e-2
    assert torch.equal(a.grad.float(), (zr > 0).float()) and torch.equal(b.grad.float(), (zr > 0).float())


def test_resnet_block_graph_fused_matches_unfused_on_gpu(nat):
    from deeplearning4j_b200 import DataType, Nd4j, nn
    from deeplearning4j_b200.data import DataSet

    def build():
        conf = (nn.NeuralNetConfiguration.Builder().seed(9).updater(nn.Sgd(0.05)).computeDataType(DataType.BFLOAT16).graphBuilder()
                .addInputs("in")
                .addLayer("c1", nn.ConvolutionLayer(kernelSize=(3, 3), padding=(1, 1), nIn=16, nOut=16, activation="identity"), "in")
                .addLayer("bn1", nn.BatchNormalization(nOut=16), "c1")
                .addLayer("r1", nn.ActivationLayer("relu"), "bn1")
                .addLayer("c2", nn.ConvolutionLayer(kernelSize=(1, 1), nIn=16, nOut=16, activation="identity"), "r1")
                .addLayer("bn2", nn.BatchNormalization(nOut=16), "c2")
                .addVertex("add", nn.ElementWiseVertex("Add"), "bn2", "in")
                .addLayer("r2", nn.ActivationLayer("relu"), "add")
                .addLayer("gp", nn.GlobalPoolingLayer("AVG"), "r2")
                .addLayer("out", nn.OutputLayer("MCXENT", nIn=16, nOut=3, activation="softmax"), "gp")
                .setOutputs("out").setInputTypes(nn.InputType.convolutional(8, 8, 16)).build())
        net = nn.ComputationGraph(conf)
        net.device = torch.device("cuda")
        net.init()
        return net
    a, b = build(), build()
    b._fuse_plan = {}
    from deeplearning4j_b200.ops import nnops
    rng = np.random.default_rng(1)
    x = Nd4j.create(rng.normal(size=(8, 16, 8, 8)).astype(np.float32))
    y = Nd4j.create(np.eye(3, dtype=np.float32)[rng.integers(0, 3, size=8)])
    launches0 = nat.LAUNCHES
    for _ in range(3):
        a.fit(DataSet(x, y))
    assert nat.LAUNCHES > launches0
    nnops.set_force_torch(True)
    try:
        for _ in range(3):
            b.fit(DataSet(x, y))
    finally:
        nnops.set_force_torch(False)
    pa, pb = a.params().numpy().astype(np.float32), b.params().numpy().astype(np.float32)
    assert np.abs(pa - pb).max() < 3e-2 * (np.abs(pb).max() + 1e-6)
