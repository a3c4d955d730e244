"""Host side of the fused gradient-sharing kernels: symmetric (peer-mapped) buffers, the context
structure handed to ``csrc/comm_kernels.cu`` and the per-step launches.

Every rank allocates its flat parameter / gradient / shadow / message buffers through
``torch.distributed._symmetric_memory`` so that each buffer has a peer-visible address on every
other GPU of the node (and a multicast address when the NVSwitch supports NVLS).  After that one
rendezvous no further host communication happens: the kernels synchronise through flags in the
signal pads.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import native

MAX_RANKS = 8


class _CommArgs(ctypes.Structure):
    _fields_ = [("rank", ctypes.c_int), ("world", ctypes.c_int),
                ("grads", ctypes.c_void_p * MAX_RANKS), ("params", ctypes.c_void_p * MAX_RANKS),
                ("shadow", ctypes.c_void_p * MAX_RANKS), ("signal", ctypes.c_void_p * MAX_RANKS),
                ("msg", ctypes.c_void_p * MAX_RANKS),
                ("mc_grads", ctypes.c_void_p), ("mc_params", ctypes.c_void_p), ("mc_shadow", ctypes.c_void_p)]


def symmetric_available() -> bool:
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
        return torch.cuda.is_available() and dist.is_initialized() and dist.get_backend() == "nccl"
    except Exception:
        return False


class SymmetricAllocator:
    """Allocates tensors in symmetric memory and remembers their rendezvous handles."""

    def __init__(self, group=None):
        import torch.distributed._symmetric_memory as symm
        self.symm = symm
        self.group = group or dist.group.WORLD
        self.handles = {}

    def empty(self, numel, dtype, device):
        t = self.symm.empty(max(int(numel), 1), dtype=dtype, device=device)
        t.zero_()
        return t

    def handle(self, t):
        key = t.untyped_storage().data_ptr()
        h = self.handles.get(key)
        if h is None:
            base = t if t.storage_offset() == 0 else t
            h = self.symm.rendezvous(base, self.group)
            self.handles[key] = h
        return h


_STATUS_NAMES = {1: "TMA producer wait", 2: "MMA wait", 3: "epilogue wait", 4: "peer wait", 5: "index out of bounds"}


class DeviceStatusPoller:
    """Surfaces the device status word (bounded waits that gave up) in the training path without a device sync.

    After every fused launch ``snapshot()`` queues a 4-byte copy of the word into pinned memory and records an event;
    ``check()`` (called before the next launch, and by ``ElasticTrainer`` at heartbeat time) reads the value once the
    event has completed.  A non-zero value means the kernel skipped its update *and* left the gradients uncleared, so the
    poller zeroes the gradient buffer, clears the word (it is sticky: every later bounded wait would bail out at once) and
    raises ``PeerFailure`` (peer wait) or ``StepTimeout`` (any other bounded wait)."""

    def __init__(self, grads=None):
        self.grads = grads
        self._pending = None        # (event, pinned tensor)
        self._pinned = None

    # -- device access, overridable in host-only tests -----------------------------------------------------------
    def _queue_copy(self):
        lib = native.require()
        if self._pinned is None:
            self._pinned = torch.zeros(1, dtype=torch.int32).pin_memory()
            lib.dl4j_status_snapshot.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
            lib.dl4j_status_snapshot.restype = ctypes.c_int
        rc = lib.dl4j_status_snapshot(ctypes.c_void_p(self._pinned.data_ptr()), native._stream())
        native._check(rc, "dl4j_status_snapshot")
        ev = torch.cuda.Event()
        ev.record()
        return ev, self._pinned

    def _clear_word(self):
        native.require().dl4j_read_status(1)

    # -------------------------------------------------------------------------------------------------------------
    def snapshot(self):
        self._pending = self._queue_copy()

    def check(self, wait=False):
        if self._pending is None:
            return 0
        ev, pinned = self._pending
        if wait:
            ev.synchronize()
        elif not ev.query():
            return 0
        self._pending = None
        v = int(pinned[0])
        if v == 0:
            return 0
        self._clear_word()
        if self.grads is not None:
            self.grads.zero_()          # the kernel left them uncleared; the next backward must not accumulate onto them
        from .elastic import PeerFailure, StepTimeout
        what = _STATUS_NAMES.get(v, str(v))
        if v == 4:
            raise PeerFailure(-1, f"device-side {what} expired in the fused gradient exchange; the step was skipped")
        raise StepTimeout(f"device-side {what} expired; the step was skipped")


class FusedSharing:
    """Per-model state for the fused kernels (one instance per training state / network)."""

    def __init__(self, params, grads, shadow, updater, alloc: SymmetricAllocator, use_multimem=None, message_ints=0):
        self.rank, self.world = dist.get_rank(alloc.group), dist.get_world_size(alloc.group)
        if self.world > MAX_RANKS:
            raise ValueError(f"fused gradient sharing supports up to {MAX_RANKS} ranks on one node")
        self.params, self.grads, self.shadow, self.updater = params, grads, shadow, updater
        self.alloc = alloc
        dev = params.device
        hp, hg = alloc.handle(params), alloc.handle(grads)
        hs = alloc.handle(shadow) if shadow is not None else None
        self.msg = None
        hm = None
        if message_ints:
            self.msg_stride = (int(message_ints) + 63) // 64 * 64
            self.msg = alloc.empty(2 * self.msg_stride, torch.int32, dev)
            hm = alloc.handle(self.msg)
        a = _CommArgs()
        a.rank, a.world = self.rank, self.world
        for r in range(self.world):
            a.grads[r] = hg.buffer_ptrs[r]
            a.params[r] = hp.buffer_ptrs[r]
            a.shadow[r] = hs.buffer_ptrs[r] if hs is not None else None
            a.signal[r] = hg.signal_pad_ptrs[r]
            a.msg[r] = hm.buffer_ptrs[r] if hm is not None else None
        mc_ok = bool(getattr(hg, "multicast_ptr", 0)) and bool(getattr(hp, "multicast_ptr", 0)) and \
            (hs is None or bool(getattr(hs, "multicast_ptr", 0)))
        # multimem.ld_reduce / multimem.st also move the requester's own copy through the switch, so plain peer loads and
        # stores carry fewer bytes per GPU below four ranks; from four ranks on the in-switch reduction wins
        self.use_multimem = (mc_ok and self.world >= 4) if use_multimem is None else (bool(use_multimem) and mc_ok)
        a.mc_grads = hg.multicast_ptr if mc_ok else None
        a.mc_params = hp.multicast_ptr if mc_ok else None
        a.mc_shadow = hs.multicast_ptr if (mc_ok and hs is not None) else None
        self.args = a
        self._handles = (hp, hg, hs, hm)
        self.scratch = torch.zeros(64, dtype=torch.int32, device=dev)
        self.status = DeviceStatusPoller(grads)
        self.epoch = 0
        self.residual = None
        lib = native.require()
        vp, i32, i64, u32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_uint, ctypes.c_float
        lib.dl4j_allreduce_update.argtypes = [vp, vp, vp, i32, vp, vp, i32, f32, i64, u32, vp, i32, vp]
        lib.dl4j_allreduce_update.restype = i32
        lib.dl4j_threshold_share.argtypes = [vp, vp, vp, vp, i32, vp, vp, i32, f32, f32, i64, u32, vp, i32, i64, vp]
        lib.dl4j_threshold_share.restype = i32
        lib.dl4j_shadow_refresh.argtypes = [vp, vp, vp, i32, vp, vp]
        lib.dl4j_shadow_refresh.restype = i32
        self.lib = lib
        # signal pads start zeroed; make sure every rank is set up before the first kernel touches a peer
        dist.barrier(group=alloc.group)

    def allreduce_update(self, iteration, epoch):
        """Dense averaging: mean gradient over ranks -> updater -> new parameters on every rank."""
        upd = self.updater
        t = native.update_tables(upd, iteration, epoch, upd.shadow_offsets)
        if t is None:
            raise RuntimeError("updater configuration is not supported by the fused kernel")
        self.status.check()               # outcome of the previous step's launch (raises PeerFailure / StepTimeout)
        self.epoch += 1
        hp = t["hyper"].ctypes.data_as(ctypes.c_void_p)
        st = upd.state
        rc = self.lib.dl4j_allreduce_update(ctypes.byref(self.args), native._ptr(st) if st.numel() else None,
                                            native._ptr(t["chunks"]), t["n_chunks"], native._ptr(t["segs_dev"]), hp, t["n_hyper"],
                                            1.0 / self.world, self.params.numel(), self.epoch, native._ptr(self.scratch),
                                            1 if self.use_multimem else 0, native._stream())
        native._check(rc, "dl4j_allreduce_update")
        self.status.snapshot()
        upd._fused_zeroes_grads = True
        upd._shadow_fresh = self.shadow is not None

    def threshold_share(self, iteration, epoch, tau):
        """Shared gradients: updater -> residual -> bitmap encode -> exchange -> decode sum -> apply."""
        upd = self.updater
        t = native.update_tables(upd, iteration, epoch, upd.shadow_offsets)
        if t is None:
            raise RuntimeError("updater configuration is not supported by the fused kernel")
        if self.residual is None:
            self.residual = torch.zeros_like(self.params)
        self.status.check()
        self.epoch += 1
        hp = t["hyper"].ctypes.data_as(ctypes.c_void_p)
        st = upd.state
        rc = self.lib.dl4j_threshold_share(ctypes.byref(self.args), native._ptr(st) if st.numel() else None,
                                           native._ptr(self.residual), native._ptr(t["chunks"]), t["n_chunks"],
                                           native._ptr(t["segs_dev"]), hp, t["n_hyper"], 1.0, float(tau), self.params.numel(),
                                           self.epoch, native._ptr(self.scratch), self.epoch & 1, self.msg_stride, native._stream())
        native._check(rc, "dl4j_threshold_share")
        if self.shadow is not None:
            rc = self.lib.dl4j_shadow_refresh(native._ptr(self.params), native._ptr(self.shadow), native._ptr(t["chunks"]),
                                              t["n_chunks"], native._ptr(t["segs_dev"]), native._stream())
            native._check(rc, "dl4j_shadow_refresh")
        self.status.snapshot()
        upd._fused_zeroes_grads = True
        upd._shadow_fresh = self.shadow is not None
