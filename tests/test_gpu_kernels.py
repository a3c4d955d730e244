"""Numerics of every hand-written CUDA kernel against a plain PyTorch fp32 reference."""
import math

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


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 192), (384, 136, 328), (1000, 776, 520), (64, 72, 40)])
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_layouts(nat, a_mn, b_mn, shape, bn):
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K + a_mn * 2 + b_mn)
    A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
    a = A.t().contiguous().t() if a_mn else A            # logical [M,K]; MN-major => stored [K,M]
    b = B if b_mn else B.t().contiguous().t()            # logical [K,N]; K-major => stored [N,K]
    ref = A.float() @ B.float()
    out = nat.gemm_raw(a, b, block_n=bn)
    torch.cuda.synchronize()
    nat.check_status()
    assert out.shape == (M, N)
    assert _rel(out, ref) < 2e-2, (a_mn, b_mn, shape, bn, _rel(out, ref))


@pytest.mark.parametrize("act", [0, 1, 2, 3, 4, 5, 6])
def test_gemm_epilogue(nat, act):
    M, N, K = 512, 384, 256
    g = torch.Generator(device="cuda").manual_seed(act)
    A = (torch.randn(M, K, device="cuda", generator=g) * 0.5).bfloat16()
    W = (torch.randn(N, K, device="cuda", generator=g) * 0.1).bfloat16()
    bias = torch.randn(N, device="cuda", generator=g)
    res = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    z = A.float() @ W.float().t() + bias
    f = {0: lambda v: v, 1: torch.relu, 2: lambda v: torch.nn.functional.gelu(v),
         3: lambda v: torch.nn.functional.gelu(v, approximate="tanh"), 4: torch.sigmoid, 5: torch.tanh,
         6: lambda v: v * torch.sigmoid(1.702 * v)}[act]
    ref = f(z) + res.float()
    aux = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    out = nat.gemm_raw(A, W.t(), bias=bias, act=act, aux=aux, residual=res)
    torch.cuda.synchronize()
    assert _rel(out, ref) < 2e-2
    assert _rel(aux, z) < 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b_mn", [0, 1])
@pytest.mark.parametrize("shape,bn", [((384, 520, 192), 256), ((200, 768, 320), 128), ((16384, 768, 768), 256)])
def test_gemm_bias_in_operand_format_is_added_on_the_tensor_core(nat, dtype, b_mn, shape, bn):
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(N + b_mn)
    A = (torch.randn(M, K, device="cuda", generator=g) * 0.5).to(dtype)
    B = (torch.randn(K, N, device="cuda", generator=g) * 0.1).to(dtype)
    b = B if b_mn else B.t().contiguous().t()
    bias = (torch.randn(N, device="cuda", generator=g) * 3).to(dtype)
    z = A.float() @ B.float() + bias.float()
    aux = torch.empty(M, N, device="cuda", dtype=dtype)
    out = nat.gemm_raw(A, b, bias=bias, act=1, aux=aux, block_n=bn)
    torch.cuda.synchronize()
    nat.check_status()
    assert _rel(aux, z) < 1e-2
    assert _rel(out, torch.relu(z)) < 1e-2


def test_gemm_fp32_out_splitk_atomic(nat):
    M, N, K = 256, 512, 4096
    g = torch.Generator(device="cuda").manual_seed(5)
    A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
    out = torch.ones(M, N, device="cuda")
    nat.gemm_raw(A, B, out=out, atomic=True, splits=8)
    ref = A.float() @ B.float() + 1.0
    torch.cuda.synchronize()
    assert _rel(out, ref) < 1e-2


def test_gemm_fp16(nat):
    A = torch.randn(256, 128, device="cuda").half()
    B = torch.randn(128, 256, device="cuda").half()
    out = nat.gemm_raw(A, B)
    assert _rel(out, A.float() @ B.float()) < 1e-2


def test_linear_autograd(nat):
    from deeplearning4j_b200.nn.activations import Activation
    M, nIn, nOut = 256, 128, 192
    x = torch.randn(M, nIn, device="cuda").bfloat16().requires_grad_(True)
    Wm = (torch.randn(nOut, nIn, device="cuda") * 0.1)
    W = Wm.t().detach().requires_grad_(True)             # logical [nIn,nOut], DL4J 'f' layout
    W.grad = torch.zeros(nOut, nIn, device="cuda").t()
    b = torch.randn(1, nOut, device="cuda").requires_grad_(True)
    b.grad = torch.zeros_like(b)
    for name in ("IDENTITY", "RELU", "GELU", "TANH"):
        act = Activation.get(name)
        W.grad.zero_(); b.grad.zero_(); x.grad = None
        y = nat.linear(x, W, b, act)
        assert y is not None
        dy = torch.randn_like(y)
        y.backward(dy)
        xr = x.detach().float().requires_grad_(True)
        Wr = W.detach().float().bfloat16().float().requires_grad_(True)
        br = b.detach().clone().requires_grad_(True)
        yr = act(xr @ Wr + br)
        yr.backward(dy.float())
        torch.cuda.synchronize()
        assert _rel(y, yr) < 2e-2, name
        assert _rel(x.grad, xr.grad) < 3e-2, name
        assert _rel(W.grad, Wr.grad) < 3e-2, name
        assert _rel(b.grad, br.grad) < 3e-2, name


@pytest.mark.parametrize("nIn,nOut", [(77, 256), (256, 77), (77, 10)])
def test_linear_with_widths_off_the_vector_grid(nat, nIn, nOut):
    """Widths that are not multiples of 8 run on the fused path through zero padding; values and all three gradients must match."""
    from deeplearning4j_b200.nn.activations import Activation
    M = 512
    g = torch.Generator(device="cuda").manual_seed(nIn * 1000 + nOut)
    x = torch.randn(M, nIn, device="cuda", generator=g).bfloat16().requires_grad_(True)
    W = (torch.randn(nOut, nIn, device="cuda", generator=g) * 0.1).t().detach().requires_grad_(True)   # logical [nIn, nOut], 'f' layout
    b = torch.randn(1, nOut, device="cuda", generator=g).requires_grad_(True)
    for name in ("IDENTITY", "TANH"):
        act = Activation.get(name)
        x.grad = W.grad = b.grad = None
        before = nat.LAUNCHES
        y = nat.linear(x, W, b, act)
        assert y is not None and y.shape == (M, nOut) and nat.LAUNCHES > before
        dy = torch.randn(M, nOut, device="cuda", generator=g).bfloat16()
        y.backward(dy)
        xr = x.detach().float().requires_grad_(True)
        Wr = W.detach().float().bfloat16().float().requires_grad_(True)
        br = b.detach().clone().requires_grad_(True)
        yr = act(xr @ Wr + br)
        yr.backward(dy.float())
        torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(x.grad.float(), xr.grad, rtol=3e-2, atol=3e-2)
        # sums over 512 rows of O(1) products: magnitudes around 20, bf16 rounding of the result alone is about 0.1
        torch.testing.assert_close(W.grad.float(), Wr.grad, rtol=3e-2, atol=0.3)
        torch.testing.assert_close(b.grad.float(), br.grad, rtol=3e-2, atol=0.3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("R,C", [(300, 768), (4100, 768), (2050, 264)])       # small and large row counts take different backward kernels
def test_layer_norm(nat, dtype, R, C):
    x = torch.randn(R, C, device="cuda").to(dtype).requires_grad_(True)
    g = torch.randn(C, device="cuda").requires_grad_(True)
    b = torch.randn(C, device="cuda").requires_grad_(True)
    y = nat.layer_norm(x, g, b, 1e-5)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    gr, br = g.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    yr = torch.nn.functional.layer_norm(xr, (C,), gr, br, 1e-5)
    yr.backward(dy.float())
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-4
    assert _rel(y, yr) < tol
    assert _rel(x.grad, xr.grad) < tol
    assert _rel(g.grad, gr.grad) < tol
    assert _rel(b.grad, br.grad) < tol


@pytest.mark.parametrize("C", [10, 1000, 30522])
def test_softmax_xent(nat, C):
    R = 64
    z = torch.randn(R, C, device="cuda").requires_grad_(True)
    idx = torch.randint(0, C, (R,), device="cuda")
    lab = torch.nn.functional.one_hot(idx, C).float()
    for sparse in (False, True):
        z.grad = None
        loss = nat.softmax_xent(z, idx if sparse else lab, sparse)
        loss.mean().backward()
        zr = z.detach().clone().requires_grad_(True)
        lr = torch.nn.functional.cross_entropy(zr, idx, reduction="none")
        lr.mean().backward()
        assert _rel(loss, lr) < 1e-4
        assert _rel(z.grad, zr.grad) < 1e-4


def test_lstm_cell(nat):
    from deeplearning4j_b200.ops import nnops
    mb, n = 64, 256
    z = torch.randn(mb, 4 * n, device="cuda").requires_grad_(True)
    c0 = torch.randn(mb, n, device="cuda").requires_grad_(True)
    h, c = nat.lstm_cell(z, c0)
    (h.sum() + (c * c).sum()).backward()
    zr, cr = z.detach().clone().requires_grad_(True), c0.detach().clone().requires_grad_(True)
    nnops.set_force_torch(True)
    try:
        hr, c2 = nnops.lstm_cell(zr, cr)
    finally:
        nnops.set_force_torch(False)
    (hr.sum() + (c2 * c2).sum()).backward()
    assert _rel(h, hr) < 1e-4 and _rel(c, c2) < 1e-4
    assert _rel(z.grad, zr.grad) < 1e-3 and _rel(c0.grad, cr.grad) < 1e-3


def test_softmax_xent_bf16_gradient_carries_the_upstream_row_scale(nat):
    g = torch.Generator(device="cuda").manual_seed(11)
    rows, C = 96, 30528
    z = (torch.randn(rows, C, device="cuda", generator=g) * 2).bfloat16().requires_grad_(True)
    idx = torch.randint(0, C, (rows,), device="cuda", generator=g)
    w = torch.rand(rows, device="cuda", generator=g)
    loss = nat.softmax_xent(z, idx, True)
    (loss * w).sum().backward()
    z32 = z.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(z32, idx, reduction="none")
    (ref * w).sum().backward()
    assert _rel(loss, ref) < 1e-3
    assert _rel(z.grad, z32.grad) < 1e-2


def test_gather_rows_scatters_gradient_into_fp32_master(nat):
    g = torch.Generator(device="cuda").manual_seed(12)
    V, C, n = 1000, 768, 4096
    master = torch.randn(V, C, device="cuda", generator=g).requires_grad_(True)
    master.grad = torch.full((V, C), 0.5, device="cuda")
    shadow = master.detach().bfloat16().requires_grad_(True)
    shadow._master = master
    idx = torch.randint(0, V, (n,), device="cuda", generator=g)
    y = nat.gather_rows(shadow, idx)
    assert torch.equal(y, shadow.detach()[idx])
    dy = torch.randn(n, C, device="cuda", generator=g).bfloat16()
    y.backward(dy)
    ref = torch.full((V, C), 0.5, device="cuda").index_add_(0, idx, dy.float())
    assert shadow.grad is None                                  # accumulated straight into the master gradient
    assert _rel(master.grad, ref) < 1e-5
    # a table without a preallocated gradient gets an ordinary gradient
    t2 = torch.randn(V, C, device="cuda", generator=g).bfloat16().requires_grad_(True)
    nat.gather_rows(t2, idx).backward(dy)
    assert _rel(t2.grad, torch.zeros(V, C, device="cuda").index_add_(0, idx, dy.float())) < 1e-2
    nat.check_status()


@pytest.mark.parametrize("n", [1000, 65536 + 17, 3_000_001])
def test_threshold_codec(nat, n):
    from deeplearning4j_b200.parallel import codec
    g = torch.Generator().manual_seed(n)
    x = torch.randn(n, generator=g) * 1e-3
    tau = 2e-3
    x_cpu, x_gpu = x.clone(), x.clone().cuda()
    m_cpu = codec.threshold_encode(x_cpu, tau)
    m_gpu = codec.threshold_encode(x_gpu, tau)
    torch.cuda.synchronize()
    k = int(m_cpu[0])
    assert int(m_gpu[0]) == k and int(m_gpu[1]) == n and int(m_gpu[3]) == 0
    assert torch.equal(torch.sort(m_gpu[4:4 + k].cpu()).values, torch.sort(m_cpu[4:4 + k]).values)
    assert torch.equal(x_gpu.cpu(), x_cpu)
    t_cpu, t_gpu = torch.zeros(n), torch.zeros(n, device="cuda")
    codec.threshold_decode(m_cpu, t_cpu)
    codec.threshold_decode(m_gpu, t_gpu)
    assert torch.equal(t_gpu.cpu(), t_cpu)
    assert torch.allclose(t_cpu + x_cpu, x, atol=1e-7)


@pytest.mark.parametrize("n", [16, 1000, 1_000_003])
def test_bitmap_codec(nat, n):
    from deeplearning4j_b200.parallel import codec
    g = torch.Generator().manual_seed(n)
    x = torch.randn(n, generator=g) * 1e-3
    tau = 1e-3
    x_cpu, x_gpu = x.clone(), x.clone().cuda()
    m_cpu = codec.bitmap_encode(x_cpu, tau)
    m_gpu = codec.bitmap_encode(x_gpu, tau)
    torch.cuda.synchronize()
    assert torch.equal(m_gpu.cpu(), m_cpu)
    assert torch.equal(x_gpu.cpu(), x_cpu)
    t_cpu, t_gpu = torch.zeros(n), torch.zeros(n, device="cuda")
    codec.bitmap_decode(m_cpu, t_cpu)
    codec.bitmap_decode(m_gpu, t_gpu)
    assert torch.equal(t_gpu.cpu(), t_cpu)


@pytest.mark.parametrize("upd_name", ["Sgd", "Nesterovs", "Adam", "AdaMax", "Nadam", "AMSGrad", "AdaBelief", "AdaGrad", "RmsProp", "AdaDelta"])
def test_fused_update_matches_torch(nat, upd_name):
    from deeplearning4j_b200 import nn
    U = getattr(nn, upd_name)

    def make(device):
        conf = (nn.NeuralNetConfiguration.Builder().seed(7).updater(U()).l2(1e-3).weightDecay(1e-4).list()
                .layer(nn.DenseLayer(nIn=40, nOut=24, activation="tanh"))
                .layer(nn.OutputLayer("MCXENT", nIn=24, nOut=5, activation="softmax")).build())
        net = nn.MultiLayerNetwork(conf)
        net.device = torch.device(device)
        return net.init()
    cpu, gpu = make("cpu"), make("cpu")
    gpu.to("cuda")
    gpu.setParams(cpu.flat_params)
    g = torch.Generator().manual_seed(3)
    for it in range(4):
        grad = torch.randn(cpu.numParams(), generator=g) * 0.1
        cpu.flat_grads.copy_(grad); gpu.flat_grads.copy_(grad.cuda())
        cpu._ensure_updater().update(it, 0, use_fused=False)
        assert gpu._ensure_updater()._fused_update(it, 0)
    torch.cuda.synchronize()
    assert torch.allclose(gpu.flat_params.cpu(), cpu.flat_params, rtol=2e-5, atol=2e-6), upd_name
    assert torch.allclose(gpu.updater.state.cpu(), cpu.updater.state, rtol=2e-5, atol=2e-6), upd_name


def test_mlp_bf16_trains_on_gpu(nat):
    from deeplearning4j_b200 import nn, DataType
    conf = (nn.NeuralNetConfiguration.Builder().seed(1).updater(nn.Adam(1e-3)).computeDataType(DataType.BFLOAT16).list()
            .layer(nn.DenseLayer(nIn=784, nOut=512, activation="relu"))
            .layer(nn.DenseLayer(nIn=512, nOut=512, activation="relu"))
            .layer(nn.OutputLayer("MCXENT", nIn=512, nOut=16, activation="softmax")).build())
    net = nn.MultiLayerNetwork(conf)
    net.device = torch.device("cuda")
    net.init()
    g = torch.Generator().manual_seed(0)
    x = torch.rand(128, 784, generator=g).cuda()
    y = torch.nn.functional.one_hot(torch.randint(0, 16, (128,), generator=g), 16).float().cuda()
    before = nat.LAUNCHES
    s0 = None
    for i in range(40):
        net.fit(x, y)
        if i == 0:
            s0 = net.score()
    assert nat.LAUNCHES - before >= 40 * 8
    assert net.score() < 0.3 * s0, (s0, net.score())
    nat.check_status()


def _lstm_ref(zx, rw, h0, c0, reverse):
    """fp32 step loop with the DL4J gate order a|f|o|g; h is rounded to bf16 between steps like the kernel's state."""
    T, mb, n4 = zx.shape
    n = n4 // 4
    h, c = h0.float(), c0.float()
    outs = [None] * T
    for s in range(T):
        t = T - 1 - s if reverse else s
        z = zx[t].float() + h.bfloat16().float() @ rw.float()
        a, f, o, g = torch.tanh(z[:, :n]), torch.sigmoid(z[:, n:2 * n]), torch.sigmoid(z[:, 2 * n:3 * n]), torch.sigmoid(z[:, 3 * n:])
        c = f * c + g * a
        h = o * torch.tanh(c)
        outs[t] = h
    return torch.stack(outs, 0), h, c


@pytest.mark.parametrize("persistent_bwd", [True, False])
@pytest.mark.parametrize("T,mb,n,reverse", [(5, 64, 256, False), (7, 33, 128, True), (12, 128, 1024, False), (1, 16, 64, False)])
def test_lstm_sequence_kernel(nat, T, mb, n, reverse, persistent_bwd, monkeypatch):
    monkeypatch.setattr(nat._LstmSeqFn, "PERSISTENT_BACKWARD", persistent_bwd)
    g = torch.Generator(device="cuda").manual_seed(T * 100 + mb + n)
    zx = (torch.randn(T, mb, 4 * n, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_(True)
    rw_store = (torch.randn(4 * n, n, device="cuda", generator=g) / math.sqrt(n)).bfloat16()
    rw = rw_store.t().requires_grad_(True)                       # logical [n, 4n], column-major storage like the parameter view
    h0 = (torch.randn(mb, n, device="cuda", generator=g) * 0.3).bfloat16().requires_grad_(True)
    c0 = (torch.randn(mb, n, device="cuda", generator=g) * 0.3).requires_grad_(True)
    hs, h_last, c_last = nat.lstm_seq(zx, rw, h0, c0, reverse)
    torch.cuda.synchronize()
    nat.check_status()
    w = torch.randn(T, mb, n, device="cuda", generator=g)
    (hs.float() * w).sum().backward()
    torch.cuda.synchronize()
    nat.check_status()
    got = [zx.grad.clone(), rw.grad.clone(), h0.grad.clone(), c0.grad.clone()]
    for t_ in (zx, rw, h0, c0):
        t_.grad = None
    ref_hs, ref_h, ref_c = _lstm_ref(zx, rw, h0, c0, reverse)
    assert _rel(hs, ref_hs) < 2e-2, _rel(hs, ref_hs)
    assert _rel(h_last, ref_h) < 2e-2
    assert _rel(c_last, ref_c) < 2e-2
    (ref_hs * w).sum().backward()
    for name, a, b in zip(("dzx", "drw", "dh0", "dc0"), got, (zx.grad, rw.grad, h0.grad, c0.grad)):
        assert _rel(a, b) < 6e-2, (name, _rel(a, b))


def test_launch_table_override_changes_grid_not_results(nat, monkeypatch):
    from deeplearning4j_b200.utils.launch import DeviceValidator, LaunchDims
    x = torch.randn(4100, 768, device="cuda").bfloat16()
    g, b = torch.randn(768, device="cuda"), torch.randn(768, device="cuda")
    ref = nat.layer_norm(x, g, b, 1e-5)
    monkeypatch.setenv("GRID_SIZE_LAYER_NORM_FWD", "1")
    LaunchDims.reload()
    try:
        assert LaunchDims.get("LAYER_NORM_FWD").grid == 1
        out = nat.layer_norm(x, g, b, 1e-5)
        assert torch.equal(out, ref)
    finally:
        monkeypatch.delenv("GRID_SIZE_LAYER_NORM_FWD")
        LaunchDims.reload()
    assert DeviceValidator().validateTable() == {}          # every table entry fits the current device


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_layer_norm_with_fused_residual(nat, dtype):
    R, C = 4100, 768
    x = torch.randn(R, C, device="cuda").to(dtype).requires_grad_(True)
    res = torch.randn(R, C, device="cuda").to(dtype).requires_grad_(True)
    g = torch.randn(C, device="cuda").requires_grad_(True)
    b = torch.randn(C, device="cuda").requires_grad_(True)
    y = nat.layer_norm(x, g, b, 1e-5, residual=res)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, rr = x.detach().float().requires_grad_(True), res.detach().float().requires_grad_(True)
    gr, br = g.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    s = (xr + rr).to(dtype).float() if dtype == torch.bfloat16 else xr + rr      # the kernel rounds the stored sum to the io type
    yr = torch.nn.functional.layer_norm(xr + rr, (C,), gr, br, 1e-5)
    yr.backward(dy.float())
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-4
    assert _rel(y, yr) < tol
    assert _rel(x.grad, xr.grad) < tol and _rel(res.grad, rr.grad) < tol
    assert _rel(g.grad, gr.grad) < tol and _rel(b.grad, br.grad) < tol


@pytest.mark.parametrize("M,N,K", [(512, 256, 64), (300, 200, 72), (1024, 768, 768), (257, 768, 520)])
def test_gemm_on_cta_pairs_matches_fp32(nat, M, N, K):
    """cta_group::2 GEMM (256 x 256 tile per SM pair): forward, MN-major dgrad, split-K wgrad with TMA reduce-add and the
    bias-by-MMA + ReLU epilogue against fp32 matmul, including row / column tails and a K tail."""
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    W = torch.randn(N, K, device="cuda", generator=g).bfloat16()
    dY = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    b = torch.randn(N, device="cuda", generator=g).bfloat16()
    ref = A.float() @ W.float().t()
    tol = dict(rtol=2e-2, atol=2e-2 * float(ref.abs().mean()))
    torch.testing.assert_close(nat.gemm_raw(A, W.t(), pair=True).float(), ref, **tol)
    torch.testing.assert_close(nat.gemm_raw(A, W.t(), bias=b, act=1, pair=True).float(), torch.relu(ref + b.float()), **tol)
    rd = dY.float() @ W.float()
    torch.testing.assert_close(nat.gemm_raw(dY, W, pair=True).float(), rd, rtol=2e-2, atol=2e-2 * float(rd.abs().mean()))
    out32 = torch.full((N, K), 0.25, device="cuda")
    nat.gemm_raw(dY.t(), A, out=out32, atomic=True, splits=2, pair=True)
    rw = dY.float().t() @ A.float() + 0.25
    torch.testing.assert_close(out32, rw, rtol=1e-3, atol=1e-3 * float(rw.abs().mean()))
    torch.cuda.synchronize()
    nat.check_status()


@pytest.mark.parametrize("act_id,fn", [(6, lambda z: z * torch.sigmoid(1.702 * z)), (3, lambda z: torch.nn.functional.gelu(z, approximate="tanh")),
                                       (1, torch.relu), (5, torch.tanh)])
def test_gemm_epilogue_multiplies_by_the_activation_gradient(act_id, fn):
    """``gemm_raw(..., residual=z, res_act=id)`` = (a @ b) * act'(z), the data-gradient GEMM that writes dz directly."""
    from deeplearning4j_b200.ops import native
    native.require()
    g = torch.Generator(device="cuda").manual_seed(act_id)
    M, K, N = 300, 192, 264
    a = (torch.randn(M, K, device="cuda", generator=g) * 0.3).bfloat16()
    b = (torch.randn(K, N, device="cuda", generator=g) * 0.3).bfloat16()
    z = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    got = native.gemm_raw(a, b, residual=z, res_act=act_id)
    zf = z.float().requires_grad_(True)
    fn(zf).sum().backward()
    ref = (a.float() @ b.float()) * zf.grad
    assert _rel(got, ref) < 3e-2
    with pytest.raises(ValueError):
        native.gemm_raw(a, b, res_act=act_id)


@pytest.mark.parametrize("precise", [False, True])
def test_fused_mlp_block_matches_fp32_and_the_two_layer_path(precise):
    from deeplearning4j_b200.nn.activations import ActivationGELU
    from deeplearning4j_b200.ops import native
    native.require()
    g = torch.Generator(device="cuda").manual_seed(11)
    M, H, F_ = 384, 128, 512
    x = (torch.randn(M, H, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_(True)

    def params():
        gg = torch.Generator(device="cuda").manual_seed(12)
        W1 = (torch.randn(H, F_, device="cuda", generator=gg) * 0.1).requires_grad_(True)
        b1 = (torch.randn(F_, device="cuda", generator=gg) * 0.1).requires_grad_(True)
        W2 = (torch.randn(F_, H, device="cuda", generator=gg) * 0.1).requires_grad_(True)
        b2 = (torch.randn(H, device="cuda", generator=gg) * 0.1).requires_grad_(True)
        for p in (W1, b1, W2, b2):
            p.grad = torch.zeros_like(p)            # the kernels accumulate into existing fp32 gradients
        return W1, b1, W2, b2
    act = ActivationGELU(precise)
    dy = torch.randn(M, H, device="cuda", generator=g).bfloat16()
    W1, b1, W2, b2 = params()
    y = native.mlp(x, W1, b1, W2, b2, act)
    assert y is not None
    y.backward(dy)
    dx_fused, x.grad = x.grad.clone(), None
    V1, c1, V2, c2 = params()
    y_sep = native.linear(native.linear(x, V1, c1, act), V2, c2, None)
    y_sep.backward(dy)
    torch.cuda.synchronize()
    native.check_status()
    assert _rel(y, y_sep) < 1e-2 and _rel(dx_fused, x.grad) < 2e-2
    for a, b in ((W1, V1), (b1, c1), (W2, V2), (b2, c2)):
        assert _rel(a.grad, b.grad) < 2e-2
    # fp32 formulation
    xf = x.detach().float().requires_grad_(True)
    R1, r1, R2, r2 = (p.detach().clone().requires_grad_(True) for p in (V1, c1, V2, c2))
    z = xf @ R1 + r1
    h = torch.nn.functional.gelu(z, approximate="tanh") if precise else z * torch.sigmoid(1.702 * z)
    (h @ R2 + r2).backward(dy.float())
    assert _rel(dx_fused, xf.grad) < 4e-2
    for a, b in ((W1, R1), (b1, r1), (W2, R2), (b2, r2)):
        assert _rel(a.grad, b.grad) < 4e-2


@pytest.mark.parametrize("rows,cols", [(4096, 1024), (130, 70), (2, 2), (64, 4096)])
def test_transpose16(nat, rows, cols):
    for dt in (torch.bfloat16, torch.float16):
        m = torch.randn(rows, cols, device="cuda").to(dt)
        out = nat.transpose16(m)
        assert out.shape == (cols, rows) and out.is_contiguous()
        assert torch.equal(out, m.t().contiguous())
