"""Pointwise convolution on the tcgen05 GEMM and channels-last max pooling against PyTorch references."""
import pytest
import torch
import torch.nn.functional as F

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


@pytest.mark.parametrize("shape,cout,stride", [((4, 64, 14, 14), 256, (1, 1)), ((2, 256, 9, 7), 64, (1, 1)), ((3, 128, 14, 14), 512, (2, 2))])
@pytest.mark.parametrize("bias", [False, True])
def test_conv1x1_matches_conv2d(nat, shape, cout, stride, bias):
    g = torch.Generator(device="cuda").manual_seed(sum(shape) + cout)
    x = torch.randn(shape, device="cuda", generator=g).bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_(True)
    W = (torch.randn(cout, shape[1], 1, 1, device="cuda", generator=g) / shape[1] ** 0.5).requires_grad_(True)     # fp32 master
    W.grad = torch.zeros_like(W)
    b = torch.randn(1, cout, device="cuda", generator=g).requires_grad_(True) if bias else None
    y = nat.conv1x1(x, W, b, stride)
    assert y is not None and y.is_contiguous(memory_format=torch.channels_last)
    w = torch.randn(y.shape, device="cuda", generator=g)
    (y.float() * w).sum().backward()
    torch.cuda.synchronize()
    nat.check_status()
    got = [x.grad.clone(), W.grad.clone()] + ([b.grad.clone()] if bias else [])
    x.grad = None
    W.grad = None
    if bias:
        b.grad = None
    ref = F.conv2d(x.float(), W.bfloat16().float(), b.reshape(-1) if bias else None, stride=stride)
    assert _rel(y, ref) < 2e-2
    (ref * w).sum().backward()
    want = [x.grad, W.grad] + ([b.grad] if bias else [])
    for name, a, r in zip(("dx", "dW", "db"), got, want):
        assert _rel(a, r) < 3e-2, (name, _rel(a, r))


@pytest.mark.parametrize("shape,k,s,p", [((2, 64, 16, 16), (3, 3), (2, 2), (0, 0)), ((3, 8, 11, 9), (3, 3), (2, 2), (1, 1)),
                                         ((2, 32, 8, 8), (2, 2), (2, 2), (0, 0)), ((1, 16, 7, 7), (3, 2), (1, 2), (1, 0))])
def test_maxpool_channels_last(nat, shape, k, s, p):
    g = torch.Generator(device="cuda").manual_seed(sum(shape))
    # quantised values make ties frequent: the first maximum in scan order must receive the gradient
    x = (torch.randint(-3, 4, shape, device="cuda", generator=g).float() / 2).bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_(True)
    y = nat.maxpool2d(x, k, s, p)
    assert y is not None
    w = torch.randn(y.shape, device="cuda", generator=g).bfloat16().float()
    (y.float() * w).sum().backward()
    got = x.grad.clone()
    x.grad = None
    xr = x.detach().float().contiguous().requires_grad_(True)
    ref = F.max_pool2d(xr, k, s, p)
    assert torch.equal(y.float(), ref)
    (ref * w).sum().backward()
    assert _rel(got, xr.grad) < 1e-2


def test_rgb_stem_convolution_pads_channels(nat):
    from deeplearning4j_b200 import nn
    layer = nn.ConvolutionLayer(kernelSize=(7, 7), stride=(2, 2), padding=(3, 3), nIn=3, nOut=16, activation="identity")
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(2, 3, 32, 32, device="cuda", generator=g).bfloat16().requires_grad_(True)
    W = (torch.randn(16, 3, 7, 7, device="cuda", generator=g) * 0.1).requires_grad_(True)
    b = torch.zeros(1, 16, device="cuda").requires_grad_(True)
    y = layer.forward({"W": W, "b": b}, x, True)
    ref = F.conv2d(x.float(), W.bfloat16().float(), None, stride=2, padding=3)
    assert _rel(y, ref) < 2e-2
    y.float().sum().backward()
    assert W.grad is not None and W.grad.shape == W.shape and x.grad.shape == x.shape


def test_conv_weight_channels_last_relayout_and_gradient(nat):
    g = torch.Generator(device="cuda").manual_seed(4)
    W = torch.randn(32, 16, 3, 3, device="cuda", generator=g).requires_grad_(True)
    W.grad = torch.zeros_like(W)
    x = torch.randn(4, 16, 10, 10, device="cuda", generator=g).bfloat16().contiguous(memory_format=torch.channels_last)
    Wc = nat.conv_weight_cl(W)
    assert Wc.dtype == torch.bfloat16 and Wc.is_contiguous(memory_format=torch.channels_last)
    assert torch.equal(Wc.float(), W.detach().bfloat16().float())
    y = F.conv2d(x, Wc, None, padding=1)
    w = torch.randn(y.shape, device="cuda", generator=g).bfloat16()
    (y * w).sum().backward()
    got = W.grad.clone()
    Wr = W.detach().clone().requires_grad_(True)
    (F.conv2d(x.float(), Wr.bfloat16().float(), None, padding=1) * w.float()).sum().backward()
    assert _rel(got, Wr.grad) < 3e-2


@pytest.mark.parametrize("shape,k,pad", [((4, 3, 224, 224), 7, 3), ((3, 3, 37, 41), 7, 3), ((2, 1, 30, 30), 3, 1), ((2, 4, 33, 32), 5, 2)])
@pytest.mark.parametrize("channels_last", [False, True])
def test_stem_space_to_depth_kernel_matches_the_torch_construction(shape, k, pad, channels_last):
    import torch.nn.functional as F
    from deeplearning4j_b200.ops import native as nat
    N, C, H, W = shape
    x = torch.randn(shape, device="cuda").bfloat16()
    if channels_last:
        x = x.contiguous(memory_format=torch.channels_last)
    OH, OW = (H + 2 * pad - k) // 2 + 1, (W + 2 * pad - k) // 2 + 1
    K2 = (k + 1) // 2
    Hs, Ws = OH + K2 - 1, OW + K2 - 1
    cp = 4 * C + (-4 * C) % 8
    got = nat.stem_space_to_depth(x, (pad, pad), Hs, Ws, cp)
    assert got is not None and got.shape == (N, cp, Hs, Ws) and got.is_contiguous(memory_format=torch.channels_last)
    eh, ew = 2 * Hs - (H + 2 * pad), 2 * Ws - (W + 2 * pad)
    xp = F.pad(x, (pad, pad + max(ew, 0), pad, pad + max(eh, 0)))[:, :, :2 * Hs, :2 * Ws]
    ref = xp.reshape(N, C, Hs, 2, Ws, 2).permute(0, 3, 5, 1, 2, 4).reshape(N, 4 * C, Hs, Ws)
    ref = F.pad(ref, (0, 0, 0, 0, 0, cp - 4 * C))
    assert torch.equal(got, ref)


def _close(a, b, rtol=2e-2, atol_frac=1e-2):
    """Element-wise check with a bf16-sized tolerance: |a - b| <= atol + rtol |b| with atol a fraction of b's rms."""
    a, b = a.detach().float(), b.detach().float()
    atol = atol_frac * float(b.pow(2).mean().sqrt()) + 1e-6
    torch.testing.assert_close(a, b, rtol=rtol, atol=atol)


@pytest.mark.parametrize("N,C,H,W,O,k,pad,dil", [
    (4, 64, 14, 14, 64, (3, 3), (1, 1), (1, 1)),        # ResNet stage shape, Same
    (2, 64, 55, 55, 64, (3, 3), (1, 1), (1, 1)),        # odd extent, boxes overhang the image
    (3, 512, 7, 7, 512, (3, 3), (1, 1), (1, 1)),        # several images per box, two 256-column tiles
    (2, 128, 28, 28, 256, (3, 3), (0, 0), (1, 1)),      # Truncate: output smaller than input
    (2, 32, 17, 13, 48, (7, 7), (3, 3), (1, 1)),        # 7x7, channel counts below one 64-wide slice
    (1, 8, 9, 11, 8, (1, 7), (0, 3), (1, 1)),           # asymmetric kernel, minimal channels
    (2, 64, 20, 20, 96, (3, 3), (2, 2), (2, 2)),        # dilation 2
    (5, 256, 14, 14, 256, (3, 3), (1, 1), (1, 1)),
])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("path", ["tap", "halo"])
def test_conv2d_implicit_gemm_matches_conv2d(nat, N, C, H, W, O, k, pad, dil, dtype, path):
    """Both forms of the forward / data-gradient kernel (one input fetch per tap; one halo box per channel slice read through
    shifted descriptors) and the weight-gradient kernel against fp32 ``F.conv2d``."""
    if dtype == torch.float16 and (C > 64 or path == "halo"):
        pytest.skip("fp16 covered on the small shapes")
    g = torch.Generator(device="cuda").manual_seed(N * 1000 + C + H + O)
    x = torch.randn(N, C, H, W, device="cuda", generator=g).to(dtype).contiguous(memory_format=torch.channels_last).requires_grad_(True)
    Wt = (torch.randn(O, C, k[0], k[1], device="cuda", generator=g) / (C * k[0] * k[1]) ** 0.5).requires_grad_(True)   # fp32 master
    Wt.grad = torch.full_like(Wt, 0.5)               # the kernel adds into the preallocated gradient
    b = torch.randn(1, O, device="cuda", generator=g).requires_grad_(True)
    y = nat.conv2d(x, Wt, b, pad, dil, path=path)
    assert y is not None and y.is_contiguous(memory_format=torch.channels_last)
    wgt = torch.randn(y.shape, device="cuda", generator=g).to(dtype)
    (y.float() * wgt.float()).sum().backward()
    torch.cuda.synchronize()
    nat.check_status()
    got = (y.detach().clone(), x.grad.clone(), Wt.grad.clone() - 0.5, b.grad.clone())
    x.grad = None
    Wt.grad = None
    b.grad = None
    xr = x.detach().float().requires_grad_(True)
    Wr = Wt.detach().to(dtype).float().requires_grad_(True)
    br = b.detach().reshape(-1).requires_grad_(True)
    ref = F.conv2d(xr, Wr, br, padding=pad, dilation=dil)
    (ref * wgt.float()).sum().backward()
    _close(got[0], ref)
    _close(got[1], xr.grad)
    _close(got[2], Wr.grad, rtol=2e-2, atol_frac=2e-2)
    _close(got[3].reshape(-1), br.grad, rtol=2e-2, atol_frac=2e-2)


def test_conv_layer_stride1_uses_native_kernels(nat):
    """A 3x3 Same convolution layer runs on the implicit-GEMM kernels (launch counter moves, no library convolution needed)."""
    from deeplearning4j_b200 import nn
    layer = nn.ConvolutionLayer(kernelSize=(3, 3), stride=(1, 1), convolutionMode="Same", nIn=64, nOut=64, activation="identity",
                                hasBias=False)
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(2, 64, 12, 12, device="cuda", generator=g).bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_(True)
    W = (torch.randn(64, 64, 3, 3, device="cuda", generator=g) * 0.05).requires_grad_(True)
    n0 = nat.LAUNCHES
    y = layer.forward({"W": W}, x, True)
    y.float().sum().backward()
    assert nat.LAUNCHES - n0 >= 5          # weight relayout, forward, dgrad, wgrad, gradient fold
    ref = F.conv2d(x.detach().float(), W.detach().bfloat16().float(), padding=1)
    _close(y, ref)


def test_stem_space_to_depth_on_native_conv(nat):
    """7x7 stride-2 RGB stem: space-to-depth view + stride-1 native convolution with the fused filter-row K slice; input has no
    gradient (the data), so the one-kernel view builder runs too."""
    from deeplearning4j_b200 import nn
    layer = nn.ConvolutionLayer(kernelSize=(7, 7), stride=(2, 2), padding=(3, 3), nIn=3, nOut=64, activation="identity")
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(4, 3, 64, 64, device="cuda", generator=g).bfloat16()
    W = (torch.randn(64, 3, 7, 7, device="cuda", generator=g) * 0.1).requires_grad_(True)
    b = torch.randn(1, 64, device="cuda", generator=g).requires_grad_(True)
    y = layer.forward({"W": W, "b": b}, x, True)
    wgt = torch.randn(y.shape, device="cuda", generator=g).bfloat16()
    (y.float() * wgt.float()).sum().backward()
    got_w, got_b = W.grad.clone(), b.grad.clone()
    Wr = W.detach().bfloat16().float().requires_grad_(True)
    br = b.detach().reshape(-1).requires_grad_(True)
    ref = F.conv2d(x.float(), Wr, br, stride=2, padding=3)
    (ref * wgt.float()).sum().backward()
    _close(y, ref)
    _close(got_w, Wr.grad, rtol=3e-2, atol_frac=3e-2)
    _close(got_b.reshape(-1), br.grad, rtol=3e-2, atol_frac=3e-2)
