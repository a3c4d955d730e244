"""Memory-mapped files as arrays (reference: libnd4j ``mmapFile`` / ``munmapFile`` and ``helpers/mman.h``)."""
import numpy as np
import pytest
import torch

from deeplearning4j_b200 import Nd4j
from deeplearning4j_b200.utils.mmap import MappedFile, mmapFile


def test_mapped_file_round_trip(tmp_path):
    p = tmp_path / "buf.bin"
    m = mmapFile(p, 4096)
    t = m.asTensor(torch.float32, (8, 16), offset=64)
    t.copy_(torch.arange(128, dtype=torch.float32).reshape(8, 16))
    m.close()
    raw = np.fromfile(p, dtype=np.float32)
    assert raw.shape == (1024,)
    np.testing.assert_array_equal(raw[16:144], np.arange(128, dtype=np.float32))
    again = MappedFile(p, readOnly=True)
    assert again.length == 4096
    assert float(again.asTensor(torch.float32)[16 + 5]) == 5.0


def test_mapped_view_checks(tmp_path):
    m = mmapFile(tmp_path / "b.bin", 64)
    with pytest.raises(ValueError):
        m.asTensor(torch.float32, (17,))
    with pytest.raises(ValueError):
        m.asTensor(torch.float32, offset=2)
    with pytest.raises(FileNotFoundError):
        MappedFile(tmp_path / "missing.bin", readOnly=True)


def test_npy_file_mapped_in_place(tmp_path):
    p = tmp_path / "a.npy"
    np.save(p, np.arange(12, dtype=np.float32).reshape(3, 4))
    a = Nd4j.createFromNpyFile(str(p), mmap=True)
    assert tuple(a.t.shape) == (3, 4)
    a.t[1, 2] = 99.0
    del a
    assert np.load(p)[1, 2] == 99.0
