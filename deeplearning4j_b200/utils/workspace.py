"""Memory workspaces (``nd4j-api/.../linalg/api/memory``: ``MemoryWorkspace``, ``Nd4jWorkspace``,
``WorkspaceConfiguration``, ``BasicWorkspaceManager``; native twin ``libnd4j/include/memory/Workspace.h``).

A workspace is a bump allocator over one device (or host) slab: tensors created inside an active scope are
views of the slab, leaving the scope resets the offset, and the slab grows to the high-water mark learned
during the first loop (``LearningPolicy.FIRST_LOOP``) or after every loop (``OVER_TIME``).  Requests that do not
fit spill to ordinary allocations (``SpillPolicy.EXTERNAL``) or fail (``FAIL``).  Because slab views alias
memory that is reused by the next iteration, ``leverageTo`` / ``detach`` copy a tensor out.  Under the hood
the slab is a ``torch.uint8`` tensor from the caching allocator, so a steady-state training loop that allocates
its temporaries here performs no allocator calls at all.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass

import torch

from ..nd.dtype import DataType
from ..nd.ndarray import INDArray


class AllocationPolicy:
    STRICT = "STRICT"
    OVERALLOCATE = "OVERALLOCATE"


class SpillPolicy:
    FAIL = "FAIL"
    EXTERNAL = "EXTERNAL"
    REALLOCATE = "REALLOCATE"


class LearningPolicy:
    NONE = "NONE"
    FIRST_LOOP = "FIRST_LOOP"
    OVER_TIME = "OVER_TIME"


class ResetPolicy:
    BLOCK_LEFT = "BLOCK_LEFT"
    ENDOFBUFFER_REACHED = "ENDOFBUFFER_REACHED"


class MirroringPolicy:
    FULL = "FULL"
    HOST_ONLY = "HOST_ONLY"


class LocationPolicy:
    RAM = "RAM"
    MMAP = "MMAP"


@dataclass
class WorkspaceConfiguration:
    initialSize: int = 0
    maxSize: int = 0
    overallocationLimit: float = 0.3
    policyAllocation: str = AllocationPolicy.OVERALLOCATE
    policySpill: str = SpillPolicy.EXTERNAL
    policyLearning: str = LearningPolicy.FIRST_LOOP
    policyReset: str = ResetPolicy.BLOCK_LEFT
    policyMirroring: str = MirroringPolicy.FULL
    policyLocation: str = LocationPolicy.RAM
    cyclesBeforeInitialization: int = 0
    stepsNumber: int = 2

    class _B:
        def __init__(self): self.kw = {}
        def __getattr__(self, k):
            if k.startswith("_") or k == "kw":
                raise AttributeError(k)
            def s(v):
                self.kw[k] = v
                return self
            return s
        def build(self): return WorkspaceConfiguration(**self.kw)

    @staticmethod
    def builder(): return WorkspaceConfiguration._B()


_ALIGN = 256


class MemoryWorkspace:
    def __init__(self, configuration=None, id="default", device=None):
        self.conf = configuration or WorkspaceConfiguration()
        self.id = id
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.slab = None
        self.offset = 0
        self.cycle_allocations = 0           # bytes requested in the current cycle (in-slab + spilled)
        self.max_cycle = 0
        self.generation = 0
        self.cycles = 0
        self.spilled = []
        self.spilled_bytes = 0
        self._open = 0
        self._prev = None
        if self.conf.initialSize > 0:
            self._allocate(self.conf.initialSize)

    # -- bookkeeping
    def getId(self): return self.id
    def getCurrentSize(self): return 0 if self.slab is None else self.slab.numel()
    def getCurrentOffset(self): return self.offset
    def getGenerationId(self): return self.generation
    def getSpilledSize(self): return self.spilled_bytes
    def getMaxCycleAllocations(self): return self.max_cycle
    def getThisCycleAllocations(self): return self.cycle_allocations
    def isScopeActive(self): return self._open > 0
    def getWorkspaceConfiguration(self): return self.conf

    def _allocate(self, nbytes):
        nbytes = int(nbytes)
        if self.conf.maxSize and nbytes > self.conf.maxSize:
            nbytes = self.conf.maxSize
        raw = torch.empty(max(nbytes, _ALIGN) + _ALIGN, dtype=torch.uint8, device=self.device)
        skew = (-raw.data_ptr()) % _ALIGN            # host allocations are only 64-byte aligned: start the slab on a 256-byte boundary
        self._raw = raw
        self.slab = raw[skew:skew + max(nbytes, _ALIGN)]

    def initializeWorkspace(self):
        want = self.max_cycle
        if self.conf.policyAllocation == AllocationPolicy.OVERALLOCATE:
            want = int(want * (1.0 + self.conf.overallocationLimit))
        want = (want + _ALIGN - 1) // _ALIGN * _ALIGN
        if want > self.getCurrentSize():
            self._allocate(want)

    # -- allocation
    def alloc(self, shape, dtype=torch.float32, initialize=False):
        """A tensor of ``shape`` backed by the workspace slab (or spilled)."""
        dtype = dtype.to_torch() if isinstance(dtype, DataType) else dtype
        numel = 1
        for s in shape:
            numel *= int(s)
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        padded = (nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
        self.cycle_allocations += padded
        if self.slab is not None and self.offset + padded <= self.slab.numel():
            t = self.slab[self.offset:self.offset + nbytes].view(dtype).reshape(tuple(shape))
            self.offset += padded
            if initialize:
                t.zero_()
            return t
        if self.conf.policySpill == SpillPolicy.FAIL and self.slab is not None:
            raise MemoryError(f"workspace '{self.id}': request of {nbytes} bytes does not fit ({self.offset}/{self.getCurrentSize()} used)")
        t = (torch.zeros if initialize else torch.empty)(tuple(shape), dtype=dtype, device=self.device)
        self.spilled.append(t)
        self.spilled_bytes += padded
        return t

    def create(self, *shape, dtype=DataType.FLOAT): return INDArray(self.alloc(shape, dtype, True))
    def createUninitialized(self, *shape, dtype=DataType.FLOAT): return INDArray(self.alloc(shape, dtype, False))

    # -- scopes
    def notifyScopeEntered(self):
        self._open += 1
        if self._open == 1:
            self._prev = _tls.current
            _tls.current = self
            self.offset = 0
            self.cycle_allocations = 0
        return self

    def notifyScopeLeft(self):
        self._open -= 1
        if self._open > 0:
            return self
        _tls.current = self._prev
        self.cycles += 1
        self.max_cycle = max(self.max_cycle, self.cycle_allocations)
        learn = self.conf.policyLearning
        if (learn == LearningPolicy.FIRST_LOOP and self.cycles == max(self.conf.cyclesBeforeInitialization, 1)) or \
                (learn == LearningPolicy.OVER_TIME and self.cycle_allocations > self.getCurrentSize()):
            self.initializeWorkspace()
        self.offset = 0
        self.generation += 1
        self.spilled.clear()
        self.spilled_bytes = 0
        return self

    def notifyScopeBorrowed(self):
        self._prev_borrow = _tls.current
        _tls.current = self
        return self

    __enter__ = notifyScopeEntered

    def __exit__(self, *a):
        self.notifyScopeLeft()

    close = notifyScopeLeft

    def destroyWorkspace(self, extended=True):
        self.slab = None
        self.offset = self.cycle_allocations = 0
        self.spilled.clear()

    # -- moving arrays out
    @staticmethod
    def detach(arr):
        t = arr.t if isinstance(arr, INDArray) else arr
        out = t.clone()
        return INDArray(out) if isinstance(arr, INDArray) else out

    def leverageTo(self, arr, target):
        t = arr.t if isinstance(arr, INDArray) else arr
        out = target.alloc(t.shape, t.dtype)
        out.copy_(t)
        return INDArray(out) if isinstance(arr, INDArray) else out

    def contains(self, arr):
        t = arr.t if isinstance(arr, INDArray) else arr
        if self.slab is None:
            return False
        a, b = self.slab.data_ptr(), self.slab.data_ptr() + self.slab.numel()
        return a <= t.data_ptr() < b


class NativeMemoryWorkspace(MemoryWorkspace):
    """The same policies over the native arena (``csrc/arena.cu`` through ``utils/arena.py``): the slab, the bump pointer, the
    spill blocks and the learned high-water mark live in the library; tensors are zero-copy views of arena addresses.  Chosen by
    ``Nd4j.getWorkspaceManager().createNewWorkspace(..., native=True)`` or ``DL4J_NATIVE_WORKSPACES=1``."""

    def __init__(self, configuration=None, id="default", device=None):
        from .arena import DEVICE, HOST, PINNED, NativeArena
        dev = torch.device(device) if device is not None else torch.device("cpu")
        conf = configuration or WorkspaceConfiguration()
        kind = DEVICE if dev.type == "cuda" else (PINNED if conf.policyLocation == "MMAP" else HOST)
        self.arena = NativeArena(kind, 0)
        super().__init__(conf, id, dev)

    def getCurrentSize(self): return self.arena.stats()["capacity"]
    def getCurrentOffset(self): return self.arena.stats()["offset"]
    def getSpilledSize(self): return self.arena.stats()["spilledBytes"]

    def _allocate(self, nbytes):
        nbytes = int(nbytes)
        if self.conf.maxSize and nbytes > self.conf.maxSize:
            nbytes = self.conf.maxSize
        self.arena.resize(max(nbytes, _ALIGN))
        self.slab = True                 # marks "initialised" for the base class's spill-policy check

    def alloc(self, shape, dtype=torch.float32, initialize=False):
        dtype = dtype.to_torch() if isinstance(dtype, DataType) else dtype
        numel = 1
        for s_ in shape:
            numel *= int(s_)
        padded = (numel * torch.empty(0, dtype=dtype).element_size() + _ALIGN - 1) // _ALIGN * _ALIGN
        self.cycle_allocations += padded
        allow = not (self.conf.policySpill == SpillPolicy.FAIL and self.slab is not None)
        try:
            return self.arena.tensor(tuple(shape), dtype, allowSpill=allow, zero=initialize)
        except MemoryError as e:
            raise MemoryError(f"workspace '{self.id}': {e}") from None

    def notifyScopeLeft(self):
        last = self._open == 1
        super().notifyScopeLeft()        # learning policy may call _allocate -> arena.resize, which needs the cycle closed first
        return self

    def notifyScopeEntered(self):
        if self._open == 0:
            self.arena.reset()
        return super().notifyScopeEntered()

    def initializeWorkspace(self):
        self.arena.reset()
        super().initializeWorkspace()

    def destroyWorkspace(self, extended=True):
        self.arena.reset()
        self.arena.resize(0)
        self.slab = None
        self.offset = self.cycle_allocations = 0

    __enter__ = notifyScopeEntered
    close = notifyScopeLeft


class _TLS(threading.local):
    current = None


_tls = _TLS()


class _ScopeOut:
    """``scopeOutOfWorkspaces()``: temporarily no current workspace."""
    def __enter__(self):
        self.prev = _tls.current
        _tls.current = None
        return self
    def __exit__(self, *a):
        _tls.current = self.prev


class BasicWorkspaceManager:
    """Per-thread registry of named workspaces (``Nd4j.getWorkspaceManager()``)."""

    def __init__(self):
        self._tls = threading.local()
        self.defaultConfiguration = WorkspaceConfiguration()

    def _map(self):
        if not hasattr(self._tls, "ws"):
            self._tls.ws = {}
        return self._tls.ws

    def setDefaultWorkspaceConfiguration(self, c): self.defaultConfiguration = c

    def createNewWorkspace(self, configuration=None, id=None, device=None, native=None):
        import os
        if native is None:
            native = os.environ.get("DL4J_NATIVE_WORKSPACES", "0") == "1"
        cls = NativeMemoryWorkspace if native else MemoryWorkspace
        ws = cls(configuration or self.defaultConfiguration, id or f"ws-{len(self._map())}", device)
        self._map()[ws.id] = ws
        return ws

    def getWorkspaceForCurrentThread(self, configuration=None, id="default", device=None):
        if isinstance(configuration, str):
            configuration, id = None, configuration
        m = self._map()
        if id not in m:
            m[id] = MemoryWorkspace(configuration or self.defaultConfiguration, id, device)
        return m[id]

    def getAndActivateWorkspace(self, configuration=None, id="default", device=None):
        return self.getWorkspaceForCurrentThread(configuration, id, device).notifyScopeEntered()

    def checkIfWorkspaceExists(self, id): return id in self._map()
    def checkIfWorkspaceExistsAndActive(self, id): return id in self._map() and self._map()[id].isScopeActive()
    def getAllWorkspacesForCurrentThread(self): return list(self._map().values())
    def getAllWorkspacesIdsForCurrentThread(self): return list(self._map())
    def scopeOutOfWorkspaces(self): return _ScopeOut()

    def destroyWorkspace(self, ws=None):
        m = self._map()
        if ws is None:
            ws = m.get("default")
        if ws is not None:
            ws.destroyWorkspace()
            m.pop(ws.id, None)

    def destroyAllWorkspacesForCurrentThread(self):
        for ws in list(self._map().values()):
            ws.destroyWorkspace()
        self._map().clear()

    def printAllocationStatisticsForCurrentThread(self):
        lines = [f"{'Workspace':<24}{'size':>14}{'max cycle':>14}{'spilled':>12}{'generation':>12}"]
        for ws in self._map().values():
            lines.append(f"{ws.id:<24}{ws.getCurrentSize():>14}{ws.max_cycle:>14}{ws.spilled_bytes:>12}{ws.generation:>12}")
        return "\n".join(lines)


def current_workspace():
    return _tls.current


_MANAGER = BasicWorkspaceManager()


def getWorkspaceManager():
    return _MANAGER


class WorkspaceMgr:
    """``LayerWorkspaceMgr``-style mapping from array roles to workspaces (``nn/workspace/ArrayType.java``)."""
    ARRAY_TYPES = ("INPUT", "ACTIVATIONS", "ACTIVATION_GRAD", "FF_WORKING_MEM", "BP_WORKING_MEM", "RNN_FF_LOOP_WORKING_MEM",
                   "RNN_BP_LOOP_WORKING_MEM", "UPDATER_WORKING_MEM", "FF_CACHE")

    def __init__(self, device=None):
        self.device, self.map, self.scoped_out = device, {}, set()

    def setWorkspace(self, arrayType, name, conf=None):
        self.map[arrayType] = getWorkspaceManager().getWorkspaceForCurrentThread(conf, name, self.device)
        return self

    def setScopedOutFor(self, arrayType): self.scoped_out.add(arrayType); return self
    def isScopedOut(self, arrayType): return arrayType in self.scoped_out or arrayType not in self.map
    def notifyScopeEntered(self, arrayType): return self.map[arrayType].notifyScopeEntered()

    def create(self, arrayType, dtype, *shape):
        if self.isScopedOut(arrayType):
            return INDArray(torch.zeros(shape, dtype=dtype.to_torch() if isinstance(dtype, DataType) else dtype, device=self.device))
        return self.map[arrayType].create(*shape, dtype=dtype)

    def createUninitialized(self, arrayType, dtype, *shape):
        if self.isScopedOut(arrayType):
            return INDArray(torch.empty(shape, dtype=dtype.to_torch() if isinstance(dtype, DataType) else dtype, device=self.device))
        return self.map[arrayType].createUninitialized(*shape, dtype=dtype)

    def leverageTo(self, arrayType, arr):
        if self.isScopedOut(arrayType):
            return MemoryWorkspace.detach(arr)
        src = current_workspace() or self.map[arrayType]
        return src.leverageTo(arr, self.map[arrayType])

    @staticmethod
    def noWorkspaces(): return WorkspaceMgr()
