"""Op benchmark suites (libnd4j ``contrib/performance/benchmarking`` ``LightBenchmarkSuit`` / ``FullBenchmarkSuit`` with
``OpBenchmark`` + parameter spaces): each benchmark names an op of the registry, a generator of inputs for a parameter point and the
bytes / FLOPs it moves; the runner times it (CUDA events on a GPU, ``perf_counter`` on the CPU) and prints one line per point.

    python -m deeplearning4j_b200.bench.ops_suite [--suite light|full] [--device cuda|cpu] [--filter substring] [--json out.json]
"""
from __future__ import annotations

import argparse
import json
import time

import torch

import deeplearning4j_b200.samediff  # noqa: F401  (registers graph-only ops)
from ..ops import registry


class OpBenchmark:
    def __init__(self, name, op, make, space, bytes_fn=None, flops_fn=None, kwargs=None):
        self.name, self.op, self.make, self.space = name, op, make, space
        self.bytes_fn, self.flops_fn, self.kwargs = bytes_fn, flops_fn, kwargs or {}


def _t(*shape, device, dtype=torch.float32):
    return torch.randn(*shape, device=device, dtype=dtype)


def _benchmarks(full):
    sizes = [1 << 16, 1 << 20] + ([1 << 24] if full else [])
    mats = [256, 1024] + ([4096] if full else [])
    B = []
    for op in ("exp", "tanh", "sigmoid", "relu", "abs", "square"):            # transform family
        B.append(OpBenchmark(f"transform/{op}", op, lambda p, dev: [_t(p, device=dev)], sizes, bytes_fn=lambda p: 8 * p))
    for op in ("add", "multiply", "maximum"):                                # pairwise / broadcast family
        B.append(OpBenchmark(f"pairwise/{op}", op, lambda p, dev: [_t(p, device=dev), _t(p, device=dev)], sizes, bytes_fn=lambda p: 12 * p))
        B.append(OpBenchmark(f"broadcast/{op}", op, lambda p, dev: [_t(p, p, device=dev), _t(p, device=dev)], mats, bytes_fn=lambda p: 8 * p * p))
    for op in ("reduce_sum", "reduce_max", "reduce_norm2"):                  # reduce family, along rows and to scalar
        B.append(OpBenchmark(f"reduce/{op}/dim1", op, lambda p, dev: [_t(p, p, device=dev)], mats, bytes_fn=lambda p: 4 * p * p,
                             kwargs={"dimensions": [1]}))
        B.append(OpBenchmark(f"reduce/{op}/all", op, lambda p, dev: [_t(p, device=dev)], sizes, bytes_fn=lambda p: 4 * p))
    B.append(OpBenchmark("index/argmax", "argmax", lambda p, dev: [_t(p, p, device=dev)], mats, bytes_fn=lambda p: 4 * p * p,
                         kwargs={"dimensions": [1]}))
    B.append(OpBenchmark("blas/matmul", "matmul", lambda p, dev: [_t(p, p, device=dev), _t(p, p, device=dev)], mats, flops_fn=lambda p: 2 * p ** 3))
    B.append(OpBenchmark("nn/softmax", "softmax", lambda p, dev: [_t(p, p, device=dev)], mats, bytes_fn=lambda p: 8 * p * p, kwargs={"dimension": 1}))
    B.append(OpBenchmark("nn/layer_norm", "layer_norm", lambda p, dev: [_t(p, p, device=dev), torch.ones(p, device=dev), torch.zeros(p, device=dev)],
                         mats, bytes_fn=lambda p: 8 * p * p))
    B.append(OpBenchmark("conv/conv2d_3x3", "conv2d", lambda p, dev: [_t(8, 32, p, p, device=dev), _t(32, 32, 3, 3, device=dev)],
                         [32, 64] + ([128] if full else []), flops_fn=lambda p: 2 * 8 * 32 * 32 * 9 * p * p,
                         kwargs={"kH": 3, "kW": 3, "pH": 1, "pW": 1, "wFormat": 1}))
    B.append(OpBenchmark("conv/maxpool2d", "maxpool2d", lambda p, dev: [_t(8, 32, p, p, device=dev)], [32, 64] + ([128] if full else []),
                         bytes_fn=lambda p: 5 * 8 * 32 * p * p))
    B.append(OpBenchmark("shape/permute", "permute", lambda p, dev: [_t(p, p, device=dev)], mats, bytes_fn=lambda p: 8 * p * p,
                         kwargs={"dimensions": [1, 0]}))
    B.append(OpBenchmark("shape/concat", "concat", lambda p, dev: [_t(p, p, device=dev), _t(p, p, device=dev)], mats, bytes_fn=lambda p: 16 * p * p,
                         kwargs={"concatDimension": 0}))
    B.append(OpBenchmark("shape/gather", "gather", lambda p, dev: [_t(p, 64, device=dev), torch.randint(0, p, (p,), device=dev)], sizes[:2],
                         bytes_fn=lambda p: 2 * 4 * 64 * p))
    if full:
        B.append(OpBenchmark("linalg/cholesky", "cholesky", lambda p, dev: [(lambda a: a @ a.t() + p * torch.eye(p, device=dev))(_t(p, p, device=dev))],
                             [256, 1024]))
        B.append(OpBenchmark("random/random_normal", "random_normal", lambda p, dev: [[p]], sizes, bytes_fn=lambda p: 4 * p, kwargs={"device": None}))
    return B


def run(suite="light", device=None, filt=None, iters=10, warmup=3):
    dev = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    rows = []
    for b in _benchmarks(suite == "full"):
        if filt and filt not in b.name:
            continue
        for p in b.space:
            ins = b.make(p, dev)
            kw = dict(b.kwargs)
            if "device" in kw:
                kw["device"] = dev
            fn = lambda: registry.execute(b.op, ins, **kw)      # noqa: E731
            for _ in range(warmup):
                fn()
            if dev.type == "cuda":
                torch.cuda.synchronize()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                for _ in range(iters):
                    fn()
                e.record()
                torch.cuda.synchronize()
                ms = s.elapsed_time(e) / iters
            else:
                t0 = time.perf_counter()
                for _ in range(iters):
                    fn()
                ms = (time.perf_counter() - t0) * 1e3 / iters
            row = {"benchmark": b.name, "param": p, "ms": ms}
            if b.bytes_fn:
                row["gbs"] = b.bytes_fn(p) / ms / 1e6
            if b.flops_fn:
                row["gflops"] = b.flops_fn(p) / ms / 1e6
            rows.append(row)
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--suite", choices=["light", "full"], default="light")
    ap.add_argument("--device", default=None)
    ap.add_argument("--filter", default=None)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default=None)
    a = ap.parse_args(argv)
    rows = run(a.suite, a.device, a.filter, a.iters)
    for r in rows:
        extra = f"{r['gbs']:9.1f} GB/s" if "gbs" in r else (f"{r['gflops']:9.1f} GFLOP/s" if "gflops" in r else "")
        print(f"{r['benchmark']:28s} {str(r['param']):>10s} {r['ms']:10.4f} ms {extra}")
    if a.json:
        with open(a.json, "w") as f:
            json.dump(rows, f, indent=1)
    return rows


if __name__ == "__main__":
    main()
