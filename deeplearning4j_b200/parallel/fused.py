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
            lib0 = native.require()
            lib0.dl4j_threshold_msg_ints.argtypes = [ctypes.c_longlong, ctypes.c_int]
            lib0.dl4j_threshold_msg_ints.restype = ctypes.c_longlong
            t0 = native.update_tables(updater, 0, 0, updater.shadow_offsets)
            if t0 is None:
                raise RuntimeError("updater configuration is not supported by the fused kernel")
            message_ints = max(int(message_ints), int(lib0.dl4j_threshold_msg_ints(params.numel(), t0["n_chunks"])))
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
        lib.dl4j_threshold_share.argtypes = [vp, vp, vp, vp, i32, vp, i32, vp, i32, f32, f32, i64, u32, vp, i32, i64, i32, vp]
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

    def average_parameters(self):
        """Classic parameter averaging (``averagingFrequency > 1``): every replica's parameters become the mean over the replicas,
        in one cooperative launch over peer memory; the bf16 shadow follows in the same kernel."""
        upd = self.updater
        t = native.update_tables(upd, 0, 0, upd.shadow_offsets)
        if t is None:
            raise RuntimeError("updater configuration is not supported by the fused kernel")
        if not hasattr(self.lib.dl4j_param_average, "_typed"):
            vp, i32, i64, u32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_uint
            self.lib.dl4j_param_average.argtypes = [vp, vp, i32, vp, i64, u32, vp, i32, vp]
            self.lib.dl4j_param_average.restype = i32
            self.lib.dl4j_param_average._typed = True
        self.status.check()
        self.epoch += 1
        rc = self.lib.dl4j_param_average(ctypes.byref(self.args), native._ptr(t["chunks"]), t["n_chunks"], native._ptr(t["segs_dev"]),
                                         self.params.numel(), self.epoch, native._ptr(self.scratch), 1 if self.use_multimem else 0,
                                         native._stream())
        native._check(rc, "dl4j_param_average")
        self.status.snapshot()
        upd._shadow_fresh = self.shadow is not None

    def threshold_share(self, iteration, epoch, tau, form=None):
        """Shared gradients in one launch: updater -> residual -> encode -> exchange -> decode sum -> apply (+ bf16 shadow).
        ``form``: 1 = bitmap, 0 = index list, None = chosen from the density the previous step reported (list when at most one
        element in 32 was sent: the list then is at most half the size of the bitmap)."""
        upd = self.updater
        t = native.update_tables(upd, iteration, epoch, upd.shadow_offsets)
        if t is None:
            raise RuntimeError("updater configuration is not supported by the fused kernel")
        if self.residual is None:
            self.residual = torch.zeros_like(self.params)
        self.status.check()
        self._poll_sent()
        if form is None:
            form = 0 if (self.last_sparsity is not None and self.last_sparsity <= 1.0 / 32.0) else 1
        self.last_form = int(form)
        self.epoch += 1
        parity = self.epoch & 1
        hp = t["hyper"].ctypes.data_as(ctypes.c_void_p)
        st = upd.state
        rc = self.lib.dl4j_threshold_share(ctypes.byref(self.args), native._ptr(st) if st.numel() else None,
                                           native._ptr(self.residual), native._ptr(t["chunks"]), t["n_chunks"],
                                           native._ptr(t["segs_dev"]), len(t["seg_rows"]), hp, t["n_hyper"], 1.0, float(tau),
                                           self.params.numel(), self.epoch, native._ptr(self.scratch), parity, self.msg_stride,
                                           int(form), native._stream())
        native._check(rc, "dl4j_threshold_share")
        # the header's element count comes back one step late (pinned copy + event, no synchronisation)
        if self._k_pinned is None:
            self._k_pinned = [torch.zeros(1, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._k_pinned[parity].copy_(self.msg[parity * self.msg_stride:parity * self.msg_stride + 1], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._k_event = (ev, parity)
        self.status.snapshot()
        upd._fused_zeroes_grads = True
        upd._shadow_fresh = self.shadow is not None

    _k_pinned = None
    _k_event = None
    last_sparsity = None
    last_form = 1

    def _poll_sent(self, wait=False):
        """Fraction of elements the last finished step sent (None until one has finished)."""
        if self._k_event is None:
            return self.last_sparsity
        ev, parity = self._k_event
        if wait:
            ev.synchronize()
        if ev.query():
            self.last_sparsity = int(self._k_pinned[parity][0]) / max(self.params.numel(), 1)
            self._k_event = None
        return self.last_sparsity


class BucketedAveraging:
    """Dense gradient averaging overlapped with the backward pass, bucket by bucket.

    The flat parameter buffer is cut into ``n_buckets`` contiguous ranges at parameter boundaries.  A parameter reports
    "gradient final" from the autograd node that presents its shadow to the graph (``samediff.training._ShadowParam``); when the
    last parameter of a bucket has reported, an event is recorded on the compute stream and ``bucket_allreduce_update_kernel``
    for that bucket is launched behind it on a side stream with a small grid, so the reduce-scatter + updater + all-gather of the
    late layers runs under the backward GEMMs of the early ones (the reference steps once, after the whole gradient is complete:
    ``optimize/solvers/StochasticGradientDescent.java:47-57``).  After backward the side stream is joined and one
    ``bucket_finish_kernel`` clears the gradients and derives the shadow of the chunks other ranks own.

    Everything that changes from step to step (Adam's bias correction, learning-rate schedule, the flag epoch) lives in a small
    device block written by ``pre_step``, so the launches can be part of a captured CUDA graph and replay unchanged.
    """

    def __init__(self, fused: FusedSharing, state, n_buckets=12, grid=32):
        self.fused, self.state = fused, state
        self.lib = fused.lib
        upd = fused.updater
        t = native.update_tables(upd, 0, 0, upd.shadow_offsets)
        if t is None:
            raise RuntimeError("updater configuration is not supported by the fused kernel")
        self.tables = t
        entries = state.entries
        total = sum(e.spec.numel for e in entries)
        n_buckets = max(1, min(int(n_buckets), len(entries), 48))
        target = total / n_buckets
        # bucket boundaries at parameter boundaries, in buffer order (= forward order); gradients become final back to front
        self.bucket_of, bounds, acc, b = {}, [0], 0, 0
        for i, e in enumerate(entries):
            self.bucket_of[e.spec.name] = b
            acc += e.spec.numel
            if acc >= target * (b + 1) and i + 1 < len(entries) and b + 1 < n_buckets:
                b += 1
                bounds.append(i + 1)
        bounds.append(len(entries))
        self.n_buckets = b + 1
        self.seg_bounds = bounds
        sc0 = upd._seg_chunk0
        self.chunk_bounds = [sc0[i] for i in bounds]
        dev = fused.params.device
        vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        self.lib.dl4j_bucket_allreduce_update.argtypes = [vp, vp, vp, i32, i32, vp, vp, i32, vp, i32, i32, vp]
        self.lib.dl4j_bucket_allreduce_update.restype = i32
        self.lib.dl4j_bucket_finish.argtypes = [vp, vp, vp, vp, i32, vp, i64, vp]
        self.lib.dl4j_bucket_finish.restype = i32
        self.lib.dl4j_step_vars_bytes.restype = i32
        self.vars_bytes = int(self.lib.dl4j_step_vars_bytes())
        self.vars_dev = torch.zeros(self.vars_bytes, dtype=torch.uint8, device=dev)
        self.tickets = torch.zeros(64, dtype=torch.int32, device=dev)
        self.bounds_dev = torch.tensor(self.chunk_bounds, dtype=torch.int32, device=dev)
        self.segs_dev = t["segs_dev"].clone()          # own copy with a fixed address (captured launches keep pointing at it)
        self._segs_key = t["segs_key"]
        import os
        self.grid = int(os.environ.get("DL4J_BUCKET_GRID", grid))
        self.side = torch.cuda.Stream(device=dev, priority=int(os.environ.get("DL4J_BUCKET_PRIO", "0")))
        self.count = [0] * self.n_buckets
        for e in entries:
            self.count[self.bucket_of[e.spec.name]] += 1
        self.pending, self.fired = list(self.count), [False] * self.n_buckets
        self.fired_early = [False] * self.n_buckets
        self.launches = 0
        for e in entries:
            leaf = state.views[e.spec.name]
            leaf._grad_ready = self._ready
            leaf._bucket = self.bucket_of[e.spec.name]

    # ------------------------------------------------------------------ per step
    def pre_step(self, iteration, epoch):
        import numpy as np
        f = self.fused
        f.status.check()
        upd = f.updater
        t = native.update_tables(upd, iteration, epoch, upd.shadow_offsets)
        if t["segs_key"] != self._segs_key:            # scheduled regularisation changed: refresh in place
            self.segs_dev.copy_(t["segs_dev"])
            self._segs_key = t["segs_key"]
        f.epoch += 1
        blob = np.zeros(self.vars_bytes, dtype=np.uint8)
        blob[:256] = np.frombuffer(t["hyper"].astype(np.float32).tobytes(), dtype=np.uint8)
        blob[256:260] = np.frombuffer(np.uint32(f.epoch).tobytes(), dtype=np.uint8)
        blob[260:264] = np.frombuffer(np.float32(1.0 / f.world).tobytes(), dtype=np.uint8)
        self.vars_dev.copy_(torch.from_numpy(blob))    # pageable source: staged at once, the buffer may be reused
        self.pending, self.fired = list(self.count), [False] * self.n_buckets
        self.fired_early = [False] * self.n_buckets     # buckets launched from a parameter's report, i.e. during backward

    def _ready(self, leaf):
        b = leaf._bucket
        self.pending[b] -= 1
        if self.pending[b] == 0 and not self.fired[b]:
            self.fired_early[b] = True
            self._fire(b)

    def _fire(self, b):
        f = self.fused
        self.fired[b] = True
        cur = torch.cuda.current_stream()
        ev = torch.cuda.Event()
        ev.record(cur)
        self.side.wait_event(ev)
        st = f.updater.state
        with torch.cuda.stream(self.side):
            rc = self.lib.dl4j_bucket_allreduce_update(ctypes.byref(f.args), native._ptr(st) if st.numel() else None,
                                                       native._ptr(self.tables["chunks"]), self.chunk_bounds[b], self.chunk_bounds[b + 1],
                                                       native._ptr(self.segs_dev), native._ptr(self.vars_dev), b, native._ptr(self.tickets),
                                                       1 if f.use_multimem else 0, self.grid, native._stream())
        native._check(rc, "dl4j_bucket_allreduce_update")

    def after_backward(self):
        f = self.fused
        for b in range(self.n_buckets - 1, -1, -1):    # whatever did not report (unused parameters): same order on every rank
            if not self.fired[b]:
                self._fire(b)
        cur = torch.cuda.current_stream()
        ev = torch.cuda.Event()
        ev.record(self.side)
        cur.wait_event(ev)
        rc = self.lib.dl4j_bucket_finish(ctypes.byref(f.args), native._ptr(self.tables["chunks"]), native._ptr(self.segs_dev),
                                         native._ptr(self.bounds_dev), self.n_buckets, native._ptr(self.vars_dev), f.params.numel(),
                                         native._stream())
        native._check(rc, "dl4j_bucket_finish")

    def __call__(self, model):
        upd = self.fused.updater
        upd._fused_zeroes_grads = True
        upd._shadow_fresh = self.fused.shadow is not None
        self.fused.status.snapshot()
        return True
