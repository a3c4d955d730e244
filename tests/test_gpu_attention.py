"""Batched tcgen05 GEMM attention vs the fp32 torch formulation."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    """Worst element-wise error in units of (|reference element| + rms of the reference): ``_rel(a, b) < t`` is
    ``allclose(a, b, rtol=t, atol=t * rms(b))`` -- a region of small values that is wrong fails, which a max-norm ratio would hide."""
    a, b = a.detach().float(), b.detach().float()
    rms = float(b.pow(2).mean().sqrt()) + 1e-12
    return float(((a - b).abs() / (b.abs() + rms)).max())


def _ref(q, k, v, mask, scale):
    s = (q.float() @ k.float().transpose(-1, -2)) * scale
    if mask is not None:
        s = s.masked_fill(mask[:, None, None, :] == 0, float("-inf"))
    return torch.softmax(s, -1) @ v.float()


@pytest.mark.parametrize("B,H,T,D", [(2, 3, 128, 64), (1, 12, 512, 64), (2, 4, 256, 64), (3, 2, 136, 32)])
@pytest.mark.parametrize("packed", [True, False])
@pytest.mark.parametrize("use_mask", [False, True])
def test_attention_fwd_bwd(B, H, T, D, packed, use_mask):
    from deeplearning4j_b200.ops import native, attention_native
    native.require()
    g = torch.Generator(device="cuda").manual_seed(B * 100 + T + D)
    if packed:
        qkv = (torch.randn(B, T, 3, H, D, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_(True)
        q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    else:
        q, k, v = ((torch.randn(B, H, T, D, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_(True) for _ in range(3))
    mask = None
    if use_mask:
        mask = (torch.rand(B, T, device="cuda", generator=g) > 0.3).float()
        mask[:, 0] = 1
    scale = D ** -0.5
    o = attention_native.attention(q, k, v, mask, scale)
    assert o is not None and o.shape == (B, H, T, D)
    do = torch.randn(B, H, T, D, device="cuda", generator=g).bfloat16()
    o.backward(do)
    torch.cuda.synchronize()
    native.check_status()
    if packed:
        qr = qkv.detach().float().requires_grad_(True)
        q2, k2, v2 = (qr[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    else:
        q2, k2, v2 = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    orf = _ref(q2, k2, v2, mask, scale)
    orf.backward(do.float())
    assert _rel(o, orf) < 3e-2
    if packed:
        assert _rel(qkv.grad, qr.grad) < 4e-2
    else:
        for a, b in ((q, q2), (k, k2), (v, v2)):
            assert _rel(a.grad, b.grad) < 4e-2


@pytest.mark.parametrize("B,H,Tq,Tk,masked", [(2, 3, 512, 512, False), (2, 2, 256, 256, True), (1, 4, 384, 512, True), (1, 1, 100, 256, False)])
def test_flash_forward_matches_reference(B, H, Tq, Tk, masked):
    from deeplearning4j_b200.ops import attention_native as an
    from deeplearning4j_b200.ops import native
    native.require()
    g = torch.Generator(device="cuda").manual_seed(B * 100 + H * 10 + Tq)
    # packed projection buffer [B, T, 3, H, 64] like the multi-head layer produces: q / k / v are strided views
    qkv = torch.randn(B, max(Tq, Tk), 3, H, 64, device="cuda", generator=g).bfloat16()
    q = qkv[:, :Tq, 0].permute(0, 2, 1, 3)
    k = qkv[:, :Tk, 1].permute(0, 2, 1, 3)
    v = qkv[:, :Tk, 2].permute(0, 2, 1, 3)
    mask = None
    if masked:
        mask = (torch.rand(B, Tk, device="cuda", generator=g) > 0.3).float()
        mask[:, 0] = 1.0
    scale = 0.125
    out, lse = an.flash_forward(q, k, v, mask, scale)
    torch.cuda.synchronize()
    native.check_status()
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale
    if mask is not None:
        s = s.masked_fill(mask[:, None, None, :] == 0, float("-inf"))
    ref = torch.matmul(torch.softmax(s, -1), v.float())                 # [B, H, Tq, 64]
    got = out.permute(0, 2, 1, 3).float()
    assert float((got - ref).abs().max()) < 2e-2 * float(ref.abs().max() + 1e-6) + 2e-2
    ref_lse = torch.logsumexp(s, -1)
    assert float((lse - ref_lse).abs().max()) < 2e-2


def _dropout_mask(an, B, H, T, p, seed):
    """The keep mask the fused kernels apply for a given seed, read back through the kernels themselves: with q = k = 0 every
    attention weight is 1 / T, and with V = 64 one-hot key selectors the output columns are the dropped weights of those keys."""
    q = torch.zeros(B, H, T, 64, device="cuda", dtype=torch.bfloat16)
    keep = torch.zeros(B, H, T, T, device="cuda", dtype=torch.bool)
    for c0 in range(0, T, 64):
        v = torch.zeros(B, H, T, 64, device="cuda", dtype=torch.bfloat16)
        v[:, :, c0:c0 + 64] = torch.eye(64, device="cuda", dtype=torch.bfloat16)
        an.set_dropout_seed(seed)
        o = an.attention(q, q, v, None, 0.125, p)
        keep[:, :, :, c0:c0 + 64] = o != 0
    return keep


@pytest.mark.parametrize("p", [0.1, 0.5])
def test_fused_attention_dropout_mask_statistics_and_reproducibility(p):
    from deeplearning4j_b200.ops import attention_native as an
    from deeplearning4j_b200.ops import native
    native.require()
    B, H, T = 2, 3, 256
    keep = _dropout_mask(an, B, H, T, p, seed=1234)
    torch.cuda.synchronize()
    native.check_status()
    n = keep.numel()
    frac = float(keep.float().mean())
    assert abs(frac - (1 - p)) < 5 * (p * (1 - p) / n) ** 0.5 + 1e-4, frac          # five standard errors
    # no structure along rows, columns, heads: every marginal is close to 1 - p
    for dim in ((0, 1, 2), (0, 1, 3), (0, 2, 3), (1, 2, 3)):
        m = keep.float().mean(dim)
        se = (p * (1 - p) / (n / m.numel())) ** 0.5
        assert float((m - (1 - p)).abs().max()) < 6 * se, (dim, float((m - (1 - p)).abs().max()), se)
    # neighbouring elements are uncorrelated
    a, b = keep[..., :-1].float() - (1 - p), keep[..., 1:].float() - (1 - p)
    assert abs(float((a * b).mean()) / (p * (1 - p))) < 0.01
    assert torch.equal(keep, _dropout_mask(an, B, H, T, p, seed=1234))               # same seed, same mask
    other = _dropout_mask(an, B, H, T, p, seed=1235)
    assert abs(float((keep == other).float().mean()) - (p * p + (1 - p) * (1 - p))) < 0.01      # another seed: independent


@pytest.mark.parametrize("masked", [False, True])
def test_fused_attention_dropout_forward_backward_against_fp32_with_the_same_mask(masked):
    from deeplearning4j_b200.ops import attention_native as an
    from deeplearning4j_b200.ops import native
    native.require()
    B, H, T, p = 2, 2, 256, 0.2
    g = torch.Generator(device="cuda").manual_seed(77)
    keep = _dropout_mask(an, B, H, T, p, seed=99).float()
    q, k, v = ((torch.randn(B, H, T, 64, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_(True) for _ in range(3))
    mask = None
    if masked:
        mask = (torch.rand(B, T, device="cuda", generator=g) > 0.3).float()
        mask[:, 0] = 1
    an.set_dropout_seed(99)
    o = an.attention(q, k, v, mask, 0.125, p)
    do = torch.randn(B, H, T, 64, device="cuda", generator=g).bfloat16()
    o.backward(do)
    torch.cuda.synchronize()
    native.check_status()
    q2, k2, v2 = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    s = (q2 @ k2.transpose(-1, -2)) * 0.125
    if mask is not None:
        s = s.masked_fill(mask[:, None, None, :] == 0, float("-inf"))
    thr = round(p * 65536)
    w = torch.softmax(s, -1) * keep * (65536.0 / (65536 - thr))
    ref = w @ v2
    ref.backward(do.float())
    assert _rel(o, ref) < 3e-2
    for a, b in ((q, q2), (k, k2), (v, v2)):
        assert _rel(a.grad, b.grad) < 4e-2


def test_dropout_seed_advances_on_the_device_between_calls():
    from deeplearning4j_b200.ops import attention_native as an
    q = torch.zeros(1, 1, 128, 64, device="cuda", dtype=torch.bfloat16)
    v = torch.zeros(1, 1, 128, 64, device="cuda", dtype=torch.bfloat16)
    v[:, :, :64] = torch.eye(64, device="cuda", dtype=torch.bfloat16)
    an.set_dropout_seed(5)
    a = an.attention(q, q, v, None, 0.125, 0.5) != 0
    b = an.attention(q, q, v, None, 0.125, 0.5) != 0
    assert not torch.equal(a, b)


@pytest.mark.parametrize("D,T", [(32, 256), (16, 128), (48, 384)])
def test_small_head_sizes_run_on_the_fused_kernels(D, T):
    from deeplearning4j_b200.ops import attention_native as an
    from deeplearning4j_b200.ops import native
    native.require()
    B, H = 2, 3
    g = torch.Generator(device="cuda").manual_seed(D + T)
    q, k, v = ((torch.randn(B, H, T, D, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_(True) for _ in range(3))
    mask = (torch.rand(B, T, device="cuda", generator=g) > 0.2).float()
    mask[:, 0] = 1
    before = native.LAUNCHES
    o = an.attention(q, k, v, mask, None)
    assert o is not None and o.shape == (B, H, T, D)
    do = torch.randn(B, H, T, D, device="cuda", generator=g).bfloat16()
    o.backward(do)
    torch.cuda.synchronize()
    native.check_status()
    q2, k2, v2 = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = _ref(q2, k2, v2, mask, D ** -0.5)
    ref.backward(do.float())
    assert _rel(o, ref) < 3e-2
    for a, b in ((q, q2), (k, k2), (v, v2)):
        assert _rel(a.grad, b.grad) < 4e-2


@pytest.mark.parametrize("T", [128, 1024, 2048])
def test_fused_attention_sequence_lengths(T):
    from deeplearning4j_b200.ops import attention_native as an
    from deeplearning4j_b200.ops import native
    native.require()
    B, H = 1, 2
    g = torch.Generator(device="cuda").manual_seed(T)
    q, k, v = ((torch.randn(B, H, T, 64, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_(True) for _ in range(3))
    assert an.flash_supported(q, k, v)
    o = an.attention(q, k, v, None, 0.125)
    do = torch.randn(B, H, T, 64, device="cuda", generator=g).bfloat16()
    o.backward(do)
    torch.cuda.synchronize()
    native.check_status()
    q2, k2, v2 = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = _ref(q2, k2, v2, None, 0.125)
    ref.backward(do.float())
    assert _rel(o, ref) < 3e-2
    for a, b in ((q, q2), (k, k2), (v, v2)):
        assert _rel(a.grad, b.grad) < 4e-2
