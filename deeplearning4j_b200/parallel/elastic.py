"""Failure detection and checkpoint-based recovery for data-parallel training.

The reference has fault *injection* (``FailureTestingListener``) and checkpoint listeners, but no recovery logic (that was the
cluster scheduler's job).  This module supplies the missing half on the host side, never by faulting a device:

* ``HeartbeatMonitor``: every rank publishes ``(iteration, wall time)`` into the process group's key-value store once per step and
  checks its peers' entries *before* launching the next step; a peer whose entry is older than ``timeout`` seconds, or that
  announced an error, raises ``PeerFailure`` on the survivors, so no collective is entered with a dead peer.
* ``CudaWatchdog``: a thread that polls a CUDA event recorded after each step; if the event does not complete within the deadline the
  training thread gets a ``StepTimeout`` at its next check (the device is never reset or trapped; bounded waits inside the kernels are
  what let the event complete).
* ``ElasticTrainer``: drives ``net.fit`` with a heartbeat check and a checkpoint every ``checkpointEvery`` iterations (through the
  standard ``CheckpointListener`` files); ``resume()`` restores the newest checkpoint so that a relaunched job (with the same or a
  smaller world) continues from the saved iteration and updater state.
"""
from __future__ import annotations

import json
import os
import threading
import time

import torch
import torch.distributed as dist


class PeerFailure(RuntimeError):
    def __init__(self, rank, reason):
        super().__init__(f"rank {rank} failed: {reason}")
        self.rank, self.reason = rank, reason


class StepTimeout(RuntimeError):
    pass


class HeartbeatMonitor:
    def __init__(self, store=None, rank=None, world=None, timeout=10.0, prefix="hb"):
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.store = store
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.timeout, self.prefix = float(timeout), prefix
        self.beat(-1)

    def _key(self, r):
        return f"{self.prefix}/{r}"

    def beat(self, iteration, error=None):
        self.store.set(self._key(self.rank), json.dumps({"it": int(iteration), "t": time.time(), "err": error}))

    def announce_failure(self, reason):
        self.beat(-2, error=str(reason))

    def peers(self):
        out = {}
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                out[r] = json.loads(self.store.get(self._key(r)).decode())
            except Exception as e:          # noqa: BLE001  (a missing key or a closed store both mean the peer is gone)
                out[r] = {"it": None, "t": 0.0, "err": f"no heartbeat entry ({type(e).__name__})"}
        return out

    def check(self, now=None):
        """Raises ``PeerFailure`` when a peer announced an error or stopped publishing heartbeats."""
        now = time.time() if now is None else now
        for r, hb in self.peers().items():
            if hb.get("err"):
                raise PeerFailure(r, hb["err"])
            if now - hb["t"] > self.timeout:
                raise PeerFailure(r, f"no heartbeat for {now - hb['t']:.1f} s (limit {self.timeout} s)")

    def wait_all(self, iteration, poll=0.01):
        """Host-side rendezvous: returns when every peer has published ``iteration`` (or raises ``PeerFailure``)."""
        while True:
            self.check()
            if all((hb["it"] is not None and hb["it"] >= iteration) for hb in self.peers().values()):
                return
            time.sleep(poll)


class CudaWatchdog:
    """Deadline on device work without touching the device: ``arm()`` records an event on the current stream, a daemon thread
    queries it; ``check()`` raises ``StepTimeout`` on the training thread when the deadline passed before the event completed."""

    def __init__(self, deadline=60.0, poll=0.05):
        self.deadline, self.poll = float(deadline), float(poll)
        self._event, self._armed_at, self._expired = None, None, False
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True, name="dl4j-cuda-watchdog")
        self._thread.start()

    def arm(self, event=None):
        if event is None and torch.cuda.is_available():
            event = torch.cuda.Event()
            event.record()
        with self._lock:
            self._event, self._armed_at, self._expired = event, time.time(), False

    def _run(self):
        while not self._stop.wait(self.poll):
            with self._lock:
                ev, t0 = self._event, self._armed_at
                if ev is None or t0 is None:
                    continue
                done = ev.query() if hasattr(ev, "query") else bool(ev())
                if done:
                    self._event = None
                elif time.time() - t0 > self.deadline:
                    self._expired = True

    def check(self):
        if self._expired:
            raise StepTimeout(f"device work did not complete within {self.deadline} s")

    def close(self):
        self._stop.set()


class ElasticTrainer:
    def __init__(self, net, checkpointDir, checkpointEvery=10, keepLast=2, heartbeatTimeout=10.0, monitor=None):
        from ..listeners.training import CheckpointListener
        self.net, self.dir = net, checkpointDir
        os.makedirs(checkpointDir, exist_ok=True)
        self.every = int(checkpointEvery)
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.monitor = monitor if monitor is not None else (HeartbeatMonitor(timeout=heartbeatTimeout) if self.world > 1 else None)
        self.ckpt = None
        if self.rank == 0:
            self.ckpt = (CheckpointListener.Builder(checkpointDir).keepLast(keepLast).saveEveryNIterations(self.every).continueExisting(True).build())

    # ------------------------------------------------------------------ recovery
    @staticmethod
    def lastCheckpointIteration(checkpointDir):
        from ..listeners.training import CheckpointListener
        cps = CheckpointListener.availableCheckpoints(checkpointDir)
        return max((c.iteration for c in cps), default=None)

    def resume(self):
        """Load the newest checkpoint (parameters, updater state, iteration / epoch counters) into ``net``; returns the iteration
        it was taken at, or None when the directory has none."""
        from ..listeners.training import CheckpointListener
        cps = CheckpointListener.availableCheckpoints(self.dir)
        if not cps:
            return None
        last = max(cps, key=lambda c: c.iteration)
        loaded = CheckpointListener.loadCheckpoint(self.dir, last.checkpointNum)
        self.net.setParams(loaded.params())
        if loaded.getUpdater() is not None and self.net.getUpdater() is not None:
            dst, src = self.net.getUpdater().getStateViewArray(), loaded.getUpdater().getStateViewArray()
            dst_t = dst.t if hasattr(dst, "toTorch") else dst
            src_t = src.t if hasattr(src, "toTorch") else src
            with torch.no_grad():
                dst_t.copy_(src_t.to(dst_t.device))
        self.net.setIterationCount(loaded.getIterationCount())
        self.net.setEpochCount(loaded.getEpochCount())
        return last.iteration

    def _check_device_status(self, wait=False):
        """Outcome of the previous step's fused gradient exchange (a bounded device-side wait that gave up): raises
        ``PeerFailure`` / ``StepTimeout``; the poller has then cleared the status word and the stale gradients."""
        hook = getattr(self.net, "gradient_hook", None)
        poller = getattr(getattr(hook, "fused", None), "status", None)
        if poller is not None:
            poller.check(wait=wait)

    # ------------------------------------------------------------------ training
    def fit(self, batches, onFailure=None):
        """Runs ``net.fit`` over ``batches`` (iterable of ``(features, labels)`` or DataSets).  Before every step the peers'
        heartbeats are checked; a local exception is announced to the peers before it propagates.  Returns the number of
        completed iterations; raises ``PeerFailure`` on the survivors of a failed peer."""
        done = 0
        try:
            for b in batches:
                it = self.net.getIterationCount()
                if self.monitor is not None:
                    # two-phase entry: publish "about to run step it", then wait until every peer has published the same (or
                    # an error).  A rank that fails between steps never publishes the next step, so no survivor enters that
                    # step's collective alone.
                    self.monitor.beat(it)
                    self.monitor.wait_all(it)
                self._check_device_status()
                if isinstance(b, (tuple, list)):
                    self.net.fit(*b)
                else:
                    self.net.fit(b)
                done += 1
                if self.ckpt is not None:
                    self.ckpt.iterationDone(self.net, self.net.getIterationCount() - 1, self.net.getEpochCount())
            self._check_device_status(wait=True)
        except PeerFailure:
            if onFailure is not None:
                onFailure(self)
            raise
        except Exception as e:          # noqa: BLE001  (tell the peers, then re-raise)
            if self.monitor is not None:
                try:
                    self.monitor.announce_failure(f"{type(e).__name__}: {e}")
                except Exception:       # noqa: BLE001
                    pass
            raise
        return done
