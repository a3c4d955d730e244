"""Per-kernel microbenchmarks with roofline fractions.

``python -m deeplearning4j_b200.bench.kernels [--kernel NAME ...] [--small] [--iters N]``

Each case is timed with CUDA events on the launching stream after warm-up, with a 256 MiB buffer
written between iterations to flush the 126 MB L2, and reported as achieved TFLOP/s or GB/s against
the measured peaks (``MEASURED_PEAKS.json`` at the repository root when present, otherwise the
fallback 6.65 TB/s and 1.59 PFLOP/s).  ``--small`` runs one modest shape per kernel with few launches,
which is the form to put under a profiler.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..ops import native


def peaks():
    here = os.path.dirname(os.path.abspath(__file__))
    p = os.path.join(here, "..", "..", "MEASURED_PEAKS.json")
    hbm, tf, src = 6650.0, 1590.0, "fallback"
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            hbm, tf, src = float(d.get("hbm_gbs", hbm)), float(d.get("bf16_tflops", tf)), "measured"
        except Exception:
            pass
    return hbm, tf, src


class Timer:
    def __init__(self, iters, warm):
        self.iters, self.warm = iters, warm
        self.flush = torch.empty(256 * 1024 * 1024 // 4, device="cuda")

    def __call__(self, fn):
        for _ in range(self.warm):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(self.iters):
            self.flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        ts.sort()
        return ts[len(ts) // 2]


def bench_gemm(t, small, rows):
    shapes = [(8192, 8192, 4096)] if small else [(16384, 768, 768), (16384, 3072, 768), (16384, 768, 3072), (16384, 2304, 768),
                                                 (2464, 30528, 768), (8192, 8192, 8192), (64, 4096, 1024)]
    for M, N, K in shapes:
        A = torch.randn(M, K, device="cuda").bfloat16()
        W = torch.randn(N, K, device="cuda").bfloat16()
        dY = torch.randn(M, N, device="cuda").bfloat16()
        bias = torch.randn(N, device="cuda")
        out32 = torch.zeros(N, K, device="cuda")
        fl = 2.0 * M * N * K
        cases = [("gemm fwd x@W^T", lambda: native.gemm_raw(A, W.t()), lambda: torch.matmul(A, W.t()))]
        if not small:
            cases += [("gemm fwd +bias+gelu", lambda: native.gemm_raw(A, W.t(), bias=bias, act=2), None),
                      ("gemm dgrad dY@W", lambda: native.gemm_raw(dY, W), lambda: torch.matmul(dY, W)),
                      ("gemm wgrad dY^T@x fp32+=", lambda: native.gemm_raw(dY.t(), A, out=out32, atomic=True, splits=native._wgrad_splits(
                          ((N + 127) // 128) * ((K + 255) // 256), M)), lambda: torch.matmul(dY.t(), A))]
        for name, ours, lib in cases:
            ms = t(ours)
            ref = t(lib) if lib is not None else None
            rows.append({"kernel": name, "shape": f"{M}x{N}x{K}", "ms": ms, "tflops": fl / ms / 1e9, "library_ms": ref,
                         "library_tflops": None if ref is None else fl / ref / 1e9})


def bench_layer_norm(t, small, rows):
    R, C = (65536, 768) if small else (16384 * 4, 768)
    x = torch.randn(R, C, device="cuda").bfloat16().requires_grad_(True)
    g = torch.ones(C, device="cuda", requires_grad=True)
    b = torch.zeros(C, device="cuda", requires_grad=True)
    dy = torch.randn(R, C, device="cuda").bfloat16()
    ms = t(lambda: native.layer_norm(x.detach(), g.detach(), b.detach(), 1e-5))
    ref = t(lambda: torch.nn.functional.layer_norm(x.detach(), (C,), g.detach().bfloat16(), b.detach().bfloat16(), 1e-5))
    rows.append({"kernel": "layer_norm fwd", "shape": f"{R}x{C} bf16", "ms": ms, "gbs": 2 * R * C * 2 / ms / 1e6, "library_ms": ref})
    y = native.layer_norm(x, g, b, 1e-5)

    def bwd():
        x.grad = g.grad = b.grad = None
        y.backward(dy, retain_graph=True)
    ms = t(bwd)
    rows.append({"kernel": "layer_norm bwd", "shape": f"{R}x{C} bf16", "ms": ms, "gbs": 3 * R * C * 2 / ms / 1e6, "library_ms": None})


def bench_softmax_xent(t, small, rows):
    R, C = (8192, 30528) if not small else (4096, 30528)
    logits = torch.randn(R, C, device="cuda").bfloat16()
    labels = torch.randint(0, C, (R,), device="cuda")
    ms = t(lambda: native.softmax_xent(logits, labels, True))
    ref = t(lambda: torch.nn.functional.cross_entropy(logits.float(), labels))
    rows.append({"kernel": "softmax_xent fwd(+grad)", "shape": f"{R}x{C} bf16", "ms": ms, "gbs": 2 * R * C * 2 / ms / 1e6, "library_ms": ref})


def bench_updater(t, small, rows):
    from .. import nn
    n_side = 4096 if small else 10240
    conf = (nn.NeuralNetConfiguration.Builder().seed(1).updater(nn.Adam(1e-3)).list()
            .layer(nn.DenseLayer(nIn=n_side, nOut=n_side, hasBias=False, activation="identity"))
            .layer(nn.LossLayer("MSE", activation="identity")).build())
    net = nn.MultiLayerNetwork(conf)
    net.device = torch.device("cuda")
    net.init()
    upd = net._ensure_updater()
    net.flat_grads.normal_()
    n = net.flat_params.numel()
    ms = t(lambda: native.fused_update(upd, 1, 0, zero_grads=False))
    rows.append({"kernel": "fused Adam update (p,g,m,v fp32)", "shape": f"{n} params", "ms": ms, "gbs": 7 * n * 4 / ms / 1e6, "library_ms": None})
    src = net.flat_grads.clone()
    msg = None

    def enc():
        net.flat_grads.copy_(src)
        native.bitmap_encode(net.flat_grads, 1.0)
    ms = t(enc)
    rows.append({"kernel": "copy + bitmap encode (tau=1 sigma)", "shape": f"{n} fp32", "ms": ms, "gbs": (4 * n * 4 + n / 4) / ms / 1e6, "library_ms": None})


def bench_lstm_cell(t, small, rows):
    mb, n = (4096, 1024)
    z = torch.randn(mb, 4 * n, device="cuda").bfloat16()
    c = torch.randn(mb, n, device="cuda")
    ms = t(lambda: native.lstm_cell(z, c))
    rows.append({"kernel": "lstm_cell fwd", "shape": f"mb={mb} n={n}", "ms": ms, "gbs": (mb * 4 * n * 2 * 2 + mb * n * (4 + 4 + 2)) / ms / 1e6, "library_ms": None})


def bench_attention(t, small, rows):
    B, H, T, D = (8, 12, 512, 64) if small else (32, 12, 512, 64)
    q, k, v = (torch.randn(B, H, T, D, device="cuda").bfloat16() for _ in range(3))
    ms = t(lambda: native.attention(q, k, v, None, D ** -0.5))
    ref = t(lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v))
    fl = 4.0 * B * H * T * T * D
    rows.append({"kernel": "attention fwd (QK^T, softmax, PV)", "shape": f"B{B} H{H} T{T} D{D}", "ms": ms, "tflops": fl / ms / 1e9,
                 "library_ms": ref, "library_tflops": fl / ref / 1e9})
    # backward through autograd on a packed [B, T, 3, H, D] projection buffer, as the multi-head layer produces it
    qkv = (torch.randn(B, T, 3, H, D, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    qq, kk, vv = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    do = torch.randn(B, H, T, D, device="cuda").bfloat16()
    o = native.attention(qq, kk, vv, None, D ** -0.5)

    def bwd():
        qkv.grad = None
        o.backward(do, retain_graph=True)
    ms_b = t(bwd)
    q2, k2, v2 = (x.detach().clone().requires_grad_(True) for x in (q, k, v))
    o2 = torch.nn.functional.scaled_dot_product_attention(q2, k2, v2)

    def bwd_ref():
        q2.grad = k2.grad = v2.grad = None
        o2.backward(do, retain_graph=True)
    ref_b = t(bwd_ref)
    rows.append({"kernel": "attention bwd (dQ, dK, dV; autograd)", "shape": f"B{B} H{H} T{T} D{D}", "ms": ms_b, "tflops": 2.5 * fl / ms_b / 1e9,
                 "library_ms": ref_b, "library_tflops": 2.5 * fl / ref_b / 1e9})


def bench_conv(t, small, rows):
    """3x3 stride-1 convolutions of the ResNet-50 stages (forward; forward + dgrad + wgrad through autograd) against cuDNN."""
    import torch.nn.functional as F
    torch.backends.cudnn.benchmark = True
    shapes = [(256, 64, 55, 64)] if small else [(256, 64, 55, 64), (256, 128, 28, 128), (256, 256, 14, 256), (256, 512, 7, 512)]
    for N, C, H, O in shapes:
        x = torch.randn(N, C, H, H, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_(True)
        W = (torch.randn(O, C, 3, 3, device="cuda") * 0.05).requires_grad_(True)
        W.grad = torch.zeros_like(W)
        Wb = W.detach().bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_(True)
        fl = 2.0 * N * H * H * C * O * 9
        ms = t(lambda: native.conv2d(x.detach(), W, None, (1, 1), (1, 1)))
        ref = t(lambda: F.conv2d(x.detach(), Wb.detach(), padding=1))
        rows.append({"kernel": "conv3x3 fwd (implicit GEMM)", "shape": f"N{N} C{C} H{H} O{O}", "ms": ms, "tflops": fl / ms / 1e9,
                     "library_ms": ref, "library_tflops": fl / ref / 1e9})
        y = native.conv2d(x, W, None, (1, 1), (1, 1))
        dy = torch.randn_like(y)

        def bwd():
            x.grad = None
            y.backward(dy, retain_graph=True)
        yl = F.conv2d(x, Wb, padding=1)

        def bwd_ref():
            x.grad = Wb.grad = None
            yl.backward(dy, retain_graph=True)
        ms_b, ref_b = t(bwd), t(bwd_ref)
        rows.append({"kernel": "conv3x3 bwd (dgrad + wgrad)", "shape": f"N{N} C{C} H{H} O{O}", "ms": ms_b, "tflops": 2 * fl / ms_b / 1e9,
                     "library_ms": ref_b, "library_tflops": 2 * fl / ref_b / 1e9})


def bench_mma_issue(t, small, rows):
    """Clocks per tcgen05.mma seen by one issuing thread, for one to four issuing warps (``csrc/mma_issue_probe.cu``).  Prints its
    own table: the figures are clock counts, not rates against a roofline."""
    import ctypes
    l = native.require()
    l.dl4j_mma_issue_probe.argtypes = [ctypes.c_int] * 6 + [ctypes.c_void_p]
    l.dl4j_mma_issue_probe.restype = ctypes.c_int
    out = (ctypes.c_longlong * 2)()
    iters = 256
    print("tcgen05.mma issue probe (M 128, bf16, K 16): clocks per instruction for each issuing thread")
    for n, issuers, mn in ((16, 1, 0), (64, 1, 0), (128, 1, 0), (256, 1, 0), (16, 4, 0), (64, 2, 0), (64, 4, 0), (128, 2, 0), (128, 4, 0),
                           (256, 2, 0), (64, 1, 1), (128, 1, 1), (256, 1, 1), (64, 4, 1), (256, 2, 1)):
        rc = l.dl4j_mma_issue_probe(128, n, iters, 1, issuers, mn, out)
        if rc != 0 or out[1] < 0:
            raise RuntimeError(f"dl4j_mma_issue_probe failed: rc {rc}, completion {out[1]}")
        per = out[1] / iters
        print(f"  N {n:3d}  {'MN' if mn else 'K '}-major  issuers {issuers}:  issue {out[0] / iters:6.1f}  complete {per:6.1f}  ->  {per / issuers:6.1f} clocks per instruction overall", flush=True)


KERNELS = {"conv": bench_conv, "mma_issue": bench_mma_issue, "gemm": bench_gemm, "layer_norm": bench_layer_norm, "softmax_xent": bench_softmax_xent, "updater": bench_updater,
           "lstm_cell": bench_lstm_cell, "attention": bench_attention}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", action="append", choices=sorted(KERNELS))
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--iters", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--json", default=None)
    a = ap.parse_args(argv)
    native.require()
    hbm, tf, src = peaks()
    t = Timer(a.iters or (2 if a.small else 15), a.warmup if a.warmup is not None else (1 if a.small else 4))
    rows = []
    for k in a.kernel or sorted(KERNELS):
        KERNELS[k](t, a.small, rows)
    torch.cuda.synchronize()
    native.check_status()
    for r in rows:
        if "tflops" in r:
            r["frac_of_peak"] = r["tflops"] / tf
            perf = f"{r['tflops']:9.1f} TFLOP/s  {100 * r['frac_of_peak']:5.1f}% of {src} {tf:.0f}"
        else:
            r["frac_of_peak"] = r["gbs"] / hbm
            perf = f"{r['gbs']:9.1f} GB/s     {100 * r['frac_of_peak']:5.1f}% of {src} {hbm:.0f}"
        lib = "" if not r.get("library_ms") else f"   library {r['library_ms']:.4f} ms"
        print(f"{r['kernel']:<36}{r['shape']:<24}{r['ms']:9.4f} ms {perf}{lib}", flush=True)
    if a.json:
        with open(a.json, "w") as f:
            json.dump({"peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src}, "rows": rows}, f, indent=1)


if __name__ == "__main__":
    main()
