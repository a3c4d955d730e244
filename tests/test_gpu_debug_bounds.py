"""The debug-bounds build of the native library (kernels check the element offsets they are about to touch, record the first
violation and skip the access) run over odd sizes: nothing may be recorded and the results must equal the normal formulation.
One case feeds a class label outside [0, C): the kernels already ignore such a label, the debug build also records it."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import sys
sys.path.insert(0, %(root)r)
import torch
import torch.nn.functional as F
from deeplearning4j_b200.ops import native
assert native._LIB_PATH.endswith("_dbg.so")
native.require()
dev = "cuda"
torch.manual_seed(3)

def close(a, b, tol):
    a, b = a.float(), b.float()
    assert float((a - b).abs().max()) <= tol * (float(b.abs().max()) + 1e-6), float((a - b).abs().max())

# layer norm over an odd number of rows and a width that is not a multiple of the per-lane vector count
for rows, C in ((37, 264), (1, 8), (513, 1000)):
    x = torch.randn(rows, C, device=dev).bfloat16().requires_grad_(True)
    g, b = torch.randn(C, device=dev).requires_grad_(True), torch.randn(C, device=dev).requires_grad_(True)
    g.grad, b.grad = torch.zeros_like(g), torch.zeros_like(b)
    y = native.layer_norm(x, g, b, 1e-5)
    y.backward(torch.randn_like(y))
    close(y, F.layer_norm(x.float(), (C,), g, b, 1e-5), 2e-2)
# pooling, subsampling and batch norm at odd spatial sizes
for N, C, H, W in ((3, 16, 13, 11), (1, 8, 7, 7), (2, 64, 57, 57)):
    x = torch.randn(N, C, H, W, device=dev).bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_(True)
    y = native.maxpool2d(x, (3, 3), (2, 2), (1, 1))
    y.backward(torch.randn_like(y))
    close(y, F.max_pool2d(x.float(), 3, 2, 1), 1e-6)
    Wt = (torch.randn(16, C, 1, 1, device=dev) * 0.1).requires_grad_(True)
    Wt.grad = torch.zeros_like(Wt)
    z = native.conv1x1(x, Wt, None, (2, 2))
    z.backward(torch.randn_like(z))
    close(z, F.conv2d(x.float(), Wt, stride=2), 3e-2)
    gamma, beta = torch.ones(C, device=dev).requires_grad_(True), torch.zeros(C, device=dev).requires_grad_(True)
    gamma.grad, beta.grad = torch.zeros_like(gamma), torch.zeros_like(beta)
    rm, rs = torch.zeros(C, device=dev), torch.ones(C, device=dev)
    o = native.bn_act_train(x, None, gamma, beta, rm, rs, False, 0.9, 1e-5, True)
    o.backward(torch.randn_like(o))
    close(o, F.relu(F.batch_norm(x.float(), None, None, gamma, beta, True, 0.1, 1e-5)), 3e-2)
# embedding gather and its scatter-add gradient
tab = torch.randn(101, 72, device=dev).requires_grad_(True)
tab.grad = torch.zeros_like(tab)
idx = torch.randint(0, 101, (7, 13), device=dev)
e = native.gather_rows(tab, idx)
e.backward(torch.randn_like(e))
torch.cuda.synchronize()
rec = native.debug_bounds()
assert rec is not None and rec["failures"] == 0, rec
assert native.check_status() == 0
# a label outside [0, C): ignored by the kernel (loss 0 for that row), recorded by the debug build, nothing touched out of range
logits = torch.randn(5, 11, device=dev).bfloat16()
labels = torch.tensor([1, 2, 99, 3, 4], device=dev)
loss = native.softmax_xent(logits, labels, True)
torch.cuda.synchronize()
rec = native.debug_bounds()
assert rec["failures"] >= 1 and rec["offset"] == 99 and rec["extent"] == 11, rec
assert native.debug_bounds()["failures"] == 0            # cleared by the read
print("DEBUG_BOUNDS_CHILD_OK")
"""


def test_debug_bounds_build_records_nothing_at_odd_sizes_and_records_a_bad_label():
    from deeplearning4j_b200.csrc import build
    if not os.path.exists(build.DEBUG_LIB):
        build.build(debug_bounds=True)
    env = dict(os.environ, DL4J_DEBUG_BOUNDS="1")
    r = subprocess.run([sys.executable, "-c", CHILD % {"root": ROOT}], capture_output=True, text=True, env=env, timeout=900)
    assert r.returncode == 0 and "DEBUG_BOUNDS_CHILD_OK" in r.stdout, (r.stdout[-1500:] + r.stderr[-3000:])
