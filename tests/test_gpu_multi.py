"""Multi-GPU tests: run the worker under torchrun on 2 GPUs of one node."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(what, n=2, port=29711, extra_env=None, timeout=600):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    env = dict(os.environ)
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "mp_fused_worker.py"), what]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    if r.returncode != 0 or "WORKER_OK" not in r.stdout:
        own = [l for l in (r.stdout + r.stderr).splitlines() if l.startswith("[rank")]
        raise AssertionError("\n".join(own[-25:]) or (r.stdout[-1500:] + r.stderr[-1500:]))
    return r.stdout


def test_fused_averaging_matches_nccl():
    _run("averaging", port=29711)


def test_fused_threshold_matches_host_codec():
    _run("threshold", port=29712)


def test_bucketed_exchange_overlapped_with_backward_matches_nccl():
    _run("bucketed", port=29714)


def test_fused_parameter_averaging_matches_the_library_path():
    _run("paramavg", port=29715)


def test_fused_paths_with_state_slots_off_the_vector_grid():
    """269,682 parameters: the second Adam state half starts 8 bytes off the 16-byte grid (the kernels move it with 4-byte accesses)."""
    _run("averaging", port=29716, extra_env={"DL4J_TEST_NOUT": "10"})
    _run("threshold", port=29717, extra_env={"DL4J_TEST_NOUT": "10"})


def test_bounded_peer_wait_reports_timeout():
    _run("timeout", port=29713, extra_env={"NCCL_NVLS_ENABLE": "0"})
