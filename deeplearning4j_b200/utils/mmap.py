"""Memory-mapped arrays (``libnd4j/include/helpers/mman.h`` + ``mmapFile`` / ``munmapFile`` of the C ABI, and the workspaces'
``LocationPolicy.MMAP``): a file region becomes an array without being read into memory; writes go back to the file."""
from __future__ import annotations

import os

import numpy as np
import torch


class MappedFile:
    """``mmapFile(path, length)``: maps (creating or growing the file when needed) ``length`` bytes read-write."""

    def __init__(self, path, length=None, readOnly=False):
        self.path = os.fspath(path)
        exists = os.path.exists(self.path)
        if not exists and readOnly:
            raise FileNotFoundError(self.path)
        size = os.path.getsize(self.path) if exists else 0
        length = size if length is None else int(length)
        if length <= 0:
            raise ValueError("cannot map an empty region")
        if not readOnly and size < length:
            with open(self.path, "ab") as f:
                f.truncate(length)
        self.length = length
        self._map = np.memmap(self.path, dtype=np.uint8, mode="r" if readOnly else "r+", shape=(length,))

    def asTensor(self, dtype=torch.float32, shape=None, offset=0):
        """A tensor over the mapped bytes starting at ``offset`` (no copy; ``shape`` defaults to everything that fits)."""
        esz = torch.empty(0, dtype=dtype).element_size()
        n = (self.length - offset) // esz if shape is None else int(np.prod(shape))
        if offset % esz or offset + n * esz > self.length:
            raise ValueError("the requested view does not fit the mapped region (or is misaligned)")
        import warnings
        with warnings.catch_warnings():                  # a read-only map yields a tensor that must not be written
            warnings.simplefilter("ignore", UserWarning)
            raw = torch.from_numpy(self._map[offset:offset + n * esz])
        t = raw.view(dtype)
        return t if shape is None else t.reshape(tuple(shape))

    def flush(self): self._map.flush()

    def close(self):
        """``munmapFile``."""
        if self._map is not None:
            self._map.flush()
            self._map = None


def mmapFile(path, length=None, readOnly=False): return MappedFile(path, length, readOnly)


def createFromNpyFileMapped(path):
    """An array over the data section of a ``.npy`` file without loading it (``Nd4j.createFromNpyFile`` with a mapped buffer)."""
    a = np.load(path, mmap_mode="r+")
    return torch.from_numpy(a)
