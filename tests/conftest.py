import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(autouse=True)
def _crash_dumps_into_tmp(tmp_path_factory):
    """Tests that make ``fit`` fail with an out-of-memory error (fault-injection listeners, the crash-dump tests) would drop their
    memory dumps into the working directory; send them to a scratch folder instead."""
    from deeplearning4j_b200.utils.crash import CrashReportingUtil
    CrashReportingUtil.crashDumpOutputDirectory(str(tmp_path_factory.getbasetemp()))
    yield
    CrashReportingUtil.crashDumpOutputDirectory(None)
