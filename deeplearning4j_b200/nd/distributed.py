"""``DistributedINDArray``: one logical array with an entry per device
(``nd4j-api/.../linalg/api/concurrency/DistributedINDArray.java:30-84``, ``BasicDistributedINDArray.java``, ``ArrayType.java``).

The reference keeps the entries of all devices in one JVM.  Here every device has its own process, so an instance is created
collectively (same calls, same order, on every rank of the group) and holds this rank's entry; with NCCL on CUDA devices the entry
lives in symmetric memory, which makes ``entry(i)`` a zero-copy view of rank ``i``'s memory over NVLink.  Without symmetric
memory (gloo ranks on CPUs) ``entry(i)`` of another rank is a collective broadcast and returns a copy.

``ArrayType`` semantics: CONSTANT entries are equal everywhere and only change through ``propagate``; SYNCABLE entries may drift
and are brought back together by ``sync`` (sum or mean over the entries); VARIADIC entries are independent (shapes may differ).
"""
from __future__ import annotations

import enum

import torch
import torch.distributed as dist

from .dtype import DataType
from .ndarray import INDArray


class ArrayType(enum.Enum):
    CONSTANT = 0
    SYNCABLE = 1
    VARIADIC = 2


def _torch_dtype(dt):
    if isinstance(dt, torch.dtype):
        return dt
    return (dt if isinstance(dt, DataType) else DataType(dt)).to_torch()


class BasicDistributedINDArray:
    def __init__(self, arrayType: ArrayType = ArrayType.SYNCABLE, group=None, device=None):
        self.arrayType = ArrayType(arrayType)
        self.group = group if group is not None else (dist.group.WORLD if dist.is_initialized() else None)
        self.rank = dist.get_rank(self.group) if self.group is not None else 0
        self.world = dist.get_world_size(self.group) if self.group is not None else 1
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        self._local = None
        self._handle = None
        self._shapes = {}                 # entry -> (shape, dtype) as allocated
        self._symmetric = (self.device.type == "cuda" and self.world > 1 and dist.is_initialized()
                           and dist.get_backend(self.group) == "nccl")

    # ------------------------------------------------------------------ interface of the reference
    def getINDArrayType(self):
        return self.arrayType

    def numEntries(self):
        return self.world

    def numActiveEntries(self):
        return len(self._shapes)

    def allocate(self, entry, dataType, *shape):
        """Collective.  Declares (and, on the owning rank, allocates) the array of ``entry``."""
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        shape, dtype = tuple(int(s) for s in shape), _torch_dtype(dataType)
        if self.arrayType is not ArrayType.VARIADIC and self._shapes and (shape, dtype) != next(iter(self._shapes.values())):
            raise ValueError(f"{self.arrayType.name} entries must share one shape and type; got {shape} after "
                             f"{next(iter(self._shapes.values()))[0]}")
        self._shapes[int(entry)] = (shape, dtype)
        if int(entry) == self.rank:
            numel = 1
            for s in shape:
                numel *= s
            if self._symmetric and self.arrayType is not ArrayType.VARIADIC:
                import torch.distributed._symmetric_memory as symm
                flat = symm.empty(max(numel, 1), dtype=dtype, device=self.device)
                flat.zero_()
                self._flat = flat
                self._local = flat[:numel].view(shape)
            else:
                self._local = torch.zeros(shape, dtype=dtype, device=self.device)
        return self

    def allocateAll(self, dataType, *shape):
        """Collective.  The same shape on every entry (what CONSTANT and SYNCABLE arrays need)."""
        for e in range(self.world):
            self.allocate(e, dataType, *shape)
        if self._symmetric and self.arrayType is not ArrayType.VARIADIC:
            import torch.distributed._symmetric_memory as symm
            self._handle = symm.rendezvous(self._flat, self.group)
        return self

    def entry(self, entry=None):
        """This rank's array, or rank ``entry``'s: a peer view when the entries are in symmetric memory, otherwise a copy obtained
        by a broadcast (collective: every rank calls ``entry(i)`` with the same ``i``)."""
        if entry is None:
            if self._local is None:
                raise KeyError(f"entry {self.rank} has not been allocated")
            return INDArray(self._local)
        entry = int(entry)
        src = entry if self.group is None or self.group is dist.group.WORLD else dist.get_global_rank(self.group, entry)
        if entry == self.rank:
            if self._local is None:
                raise KeyError(f"entry {self.rank} has not been allocated")
            if self._handle is None and self.world > 1:
                dist.broadcast(self._local, src=src, group=self.group)        # the owner's half of the peers' entry(i)
            return INDArray(self._local)
        if entry not in self._shapes:
            raise KeyError(f"entry {entry} has not been allocated")
        shape, dtype = self._shapes[entry]
        if self._handle is not None:
            numel = 1
            for s in shape:
                numel *= s
            return INDArray(self._handle.get_buffer(entry, (max(numel, 1),), dtype)[:numel].view(shape))
        buf = torch.empty(shape, dtype=dtype, device=self.device)
        dist.broadcast(buf, src=src, group=self.group)
        return INDArray(buf)

    def propagate(self, array, src=0):
        """Collective.  Every entry becomes ``array`` as held by rank ``src`` (other ranks may pass ``None``)."""
        if self.rank == src:
            t = array.t if isinstance(array, INDArray) else torch.as_tensor(array)
            meta = [tuple(t.shape), t.dtype]
        else:
            meta = [None, None]
        if self.world > 1:
            dist.broadcast_object_list(meta, src=src, group=self.group)
        shape, dtype = meta
        if not self._shapes or self._shapes.get(self.rank) != (tuple(shape), dtype):
            self._shapes.clear()
            self.allocateAll(dtype, *shape)
        if self.rank == src:
            self._local.copy_(t.to(self.device))
        if self.world > 1:
            dist.broadcast(self._local, src=src, group=self.group)
        return self

    # ------------------------------------------------------------------ SYNCABLE arrays
    def sync(self, mean=True):
        """Collective.  Replaces every entry by the sum (or mean) over all entries."""
        if self.arrayType is ArrayType.VARIADIC:
            raise ValueError("VARIADIC entries are independent; there is nothing to synchronise")
        if self.world > 1:
            dist.all_reduce(self._local, group=self.group)
            if mean:
                self._local.div_(self.world)
        return self

    def barrier(self):
        if self.world > 1:
            if self._handle is not None:
                self._handle.barrier()
            else:
                dist.barrier(group=self.group)


DistributedINDArray = BasicDistributedINDArray
