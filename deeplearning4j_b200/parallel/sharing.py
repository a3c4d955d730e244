"""Gradient sharing strategies plugged into a model's training step.

The reference's training-side data parallelism (``ParallelWrapper`` with ``AVERAGING`` /
``SHARED_GRADIENTS`` modes, ``EncodedGradientsAccumulator``, ``EncodingHandler``,
``ThresholdAlgorithm``, ``ResidualPostProcessor``) hooks in between gradient calculation and the
parameter step (``optimize/api/ConvexOptimizer.java:51``; ``StochasticGradientDescent.java:49-78``).
Here that hook is ``gradient_hook(model)``, called with the flat gradient complete.  It either
rewrites the gradient and returns False (the normal updater then runs) or performs the whole
step itself and returns True.

Implementations
  * ``NcclAveraging``      – ``all_reduce`` of the flat gradient, then the local fused updater (baseline).
  * ``FusedAveraging``     – one kernel: reduce-scatter + updater + all-gather over NVLink peer memory.
  * ``HostThresholdSharing`` – DL4J shared-gradients semantics with the host/torch codec and
    ``all_gather`` of the encoded messages; works on CPU (gloo) and as the NCCL baseline on GPU.
  * ``FusedThresholdSharing`` – one kernel: updater + residual + bitmap encode + peer exchange + decode + apply.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from . import codec


# ----------------------------------------------------------------------------- threshold algorithms
class ThresholdAlgorithm:
    def calculateThreshold(self, iteration, epoch, lastThreshold, lastWasDense, lastSparsityRatio, updates):
        raise NotImplementedError


class FixedThresholdAlgorithm(ThresholdAlgorithm):
    def __init__(self, threshold=1e-3):
        self.threshold = float(threshold)

    def calculateThreshold(self, iteration, epoch, lastThreshold, lastWasDense, lastSparsityRatio, updates):
        return self.threshold


class AdaptiveThresholdAlgorithm(ThresholdAlgorithm):
    """Keeps the encoded fraction inside [minTargetSparsity, maxTargetSparsity] by scaling the threshold
    with ``decayRate`` (historical defaults: initial 1e-3, range [1e-4, 1e-2], decay 0.965936)."""

    def __init__(self, initialThreshold=1e-3, minTargetSparsity=1e-4, maxTargetSparsity=1e-2, decayRate=0.965936):
        self.initialThreshold, self.minS, self.maxS, self.decay = float(initialThreshold), minTargetSparsity, maxTargetSparsity, decayRate

    def calculateThreshold(self, iteration, epoch, lastThreshold, lastWasDense, lastSparsityRatio, updates):
        if lastThreshold is None:
            return self.initialThreshold
        if lastWasDense or (lastSparsityRatio is not None and lastSparsityRatio > self.maxS):
            return lastThreshold / self.decay
        if lastSparsityRatio is not None and lastSparsityRatio < self.minS:
            return lastThreshold * self.decay
        return lastThreshold


class TargetSparsityThresholdAlgorithm(ThresholdAlgorithm):
    def __init__(self, initialThreshold=1e-4, sparsityTarget=1e-3, decayRate=0.965936):
        self.initialThreshold, self.target, self.decay = float(initialThreshold), sparsityTarget, decayRate

    def calculateThreshold(self, iteration, epoch, lastThreshold, lastWasDense, lastSparsityRatio, updates):
        if lastThreshold is None:
            return self.initialThreshold
        if lastSparsityRatio is None:
            return lastThreshold
        return lastThreshold / self.decay if lastSparsityRatio > self.target else lastThreshold * self.decay


class ResidualPostProcessor:
    def processResidual(self, iteration, epoch, lastThreshold, residual):
        raise NotImplementedError


class ResidualClippingPostProcessor(ResidualPostProcessor):
    """Every ``frequency`` iterations clips the residual to ``+-thresholdMultipleClipValue * threshold``."""

    def __init__(self, thresholdMultipleClipValue=5.0, frequency=5):
        self.mult, self.freq = float(thresholdMultipleClipValue), int(frequency)

    def processResidual(self, iteration, epoch, lastThreshold, residual):
        if self.freq > 0 and iteration > 0 and iteration % self.freq == 0:
            m = self.mult * lastThreshold
            residual.clamp_(-m, m)


# ----------------------------------------------------------------------------- model adapters
class _Target:
    """Uniform view of a DL4J network (``BaseNetwork``) or a SameDiff ``TrainingState``."""

    def __init__(self, model):
        self.model = model
        self.is_sd = hasattr(model, "tc")

    @property
    def params(self): return self.model.flat_params
    @property
    def grads(self): return self.model.flat_grads
    @property
    def shadow(self): return self.model.flat_shadow

    @property
    def updater(self):
        return self.model.updater if self.is_sd else self.model._ensure_updater()

    def counters(self):
        if self.is_sd:
            return self.model.tc.iterationCount, self.model.tc.epochCount
        return self.model.iterationCount, self.model.epochCount

    def refresh_shadow(self):
        self.model.refresh_shadow() if self.is_sd else self.model._refresh_shadow()


class GradientSharing:
    def __init__(self, model, group=None):
        self.t = _Target(model)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0

    def __call__(self, model):
        raise NotImplementedError

    def broadcast_parameters(self, src=0):
        """Start every replica from rank ``src``'s parameters (ParallelWrapper replicates the model)."""
        if self.world > 1:
            dist.broadcast(self.t.params, src, group=self.group)
            self.t.refresh_shadow()


class NcclAveraging(GradientSharing):
    def __call__(self, model):
        if self.world > 1:
            dist.all_reduce(self.t.grads, group=self.group)
            self.t.grads.div_(self.world)
        return False


class FusedAveraging(GradientSharing):
    def __init__(self, model, fused, group=None):
        super().__init__(model, group)
        self.fused = fused

    def __call__(self, model):
        it, ep = self.t.counters()
        self.fused.allreduce_update(it, ep)
        return True


class HostThresholdSharing(GradientSharing):
    """updater(grad) -> residual += update -> encode(residual, tau) -> all_gather -> params -= sum(decode)."""

    def __init__(self, model, thresholdAlgorithm=None, residualPostProcessor=None, group=None, encoding=None):
        super().__init__(model, group)
        self.algo = thresholdAlgorithm or AdaptiveThresholdAlgorithm(1e-3)
        self.post = residualPostProcessor
        self.residual = torch.zeros_like(self.t.params)
        self.lastThreshold, self.lastDense, self.lastSparsity = None, False, None
        self.encoding = encoding
        self.bytes_sent = 0

    def __call__(self, model):
        t = self.t
        it, ep = t.counters()
        upd = t.updater
        upd.update(it, ep, apply_step=False, use_fused=False)          # grads now hold the post-updater update
        self.residual.add_(t.grads)
        tau = self.algo.calculateThreshold(it, ep, self.lastThreshold, self.lastDense, self.lastSparsity, self.residual)
        msg = codec.encode(self.residual, tau, force=self.encoding)
        n = self.residual.numel()
        self.lastThreshold, self.lastDense = tau, int(msg[3]) == codec.BITMAP_ENCODING
        self.lastSparsity = float(msg[0]) / max(n, 1)
        if self.post is not None:
            self.post.processResidual(it, ep, tau, self.residual)
        self.bytes_sent += msg.numel() * 4
        if self.world > 1:
            msgs = _all_gather_var(msg, self.world, self.group)
        else:
            msgs = [msg]
        agg = torch.zeros_like(self.residual)
        for m in msgs:
            codec.decode(m, agg)
        t.params.sub_(agg)
        t.grads.zero_()
        t.refresh_shadow()
        return True


def _all_gather_var(msg, world, group):
    """all_gather of variable-length int32 messages (length exchanged first, then padded payloads)."""
    ln = torch.tensor([msg.numel()], dtype=torch.int64, device=msg.device)
    lens = [torch.zeros_like(ln) for _ in range(world)]
    dist.all_gather(lens, ln, group=group)
    mx = int(max(int(l) for l in lens))
    pad = torch.zeros(mx, dtype=msg.dtype, device=msg.device)
    pad[:msg.numel()] = msg
    out = [torch.zeros_like(pad) for _ in range(world)]
    dist.all_gather(out, pad, group=group)
    return [o[:int(l)] for o, l in zip(out, lens)]


class FusedThresholdSharing(GradientSharing):
    def __init__(self, model, fused, thresholdAlgorithm=None, group=None):
        super().__init__(model, group)
        self.fused = fused
        self.algo = thresholdAlgorithm or FixedThresholdAlgorithm(1e-3)
        self.lastThreshold = None

    def __call__(self, model):
        it, ep = self.t.counters()
        f = self.fused
        # density and form of the last finished step (read back without a synchronisation, so one step late)
        sparsity = f._poll_sent()
        tau = self.algo.calculateThreshold(it, ep, self.lastThreshold, f.last_form == 1, sparsity, None)
        self.lastThreshold = tau
        f.threshold_share(it, ep, tau, self.encoding)
        return True

    encoding = None       # None = by density; codec.BITMAP_ENCODING / codec.FLEXIBLE_ENCODING force a form


def attach_gradient_sharing(model, mode="averaging", impl="auto", thresholdAlgorithm=None, residualPostProcessor=None,
                            group=None, use_multimem=None, buckets=None):
    """Install a sharing strategy on ``model`` (a DL4J network or a SameDiff ``TrainingState``).

    mode: ``"averaging"`` | ``"shared_gradients"``; impl: ``"fused"`` (NVLink kernels), ``"nccl"`` / ``"host"``
    (library collectives), ``"auto"`` = fused when CUDA symmetric memory is available.
    """
    from .fused import FusedSharing, SymmetricAllocator, symmetric_available
    t = _Target(model)
    on_gpu = t.params.is_cuda
    if impl == "auto":
        impl = "fused" if (on_gpu and symmetric_available()) else "host"
    if impl == "fused" and getattr(t.updater, "needs_pre_apply", lambda: False)():
        # per-layer gradient normalisation / clipping acts on the reduced gradient before the updater; the fused kernels do not
        # do that, so such networks take the library collectives, which keep the normalisation
        impl = "nccl" if mode == "averaging" else "host"
    if impl == "fused":
        alloc = SymmetricAllocator(group)
        _rehome(model, alloc)
        t = _Target(model)
        n = t.params.numel()
        fused = FusedSharing(t.params, t.grads, t.shadow, t.updater, alloc, use_multimem,
                             message_ints=(4 + (n + 15) // 16) if mode != "averaging" else 0)
        import os
        if buckets is None:
            # default: one whole-buffer kernel after backward.  The bucketed form was measured slower on BERT-base (2 GPUs:
            # 17.4 ms/step against 16.7): a tcgen05 GEMM CTA leaves room for about 12 K registers and 1.7 KB of shared memory on its
            # SM, so the 512-thread exchange CTAs only run between GEMM launches, where they add their own launch and flag latency;
            # 128-thread CTAs that do fit next to a GEMM CTA keep too few bytes in flight over NVLink (20.2 - 34.3 ms/step).
            buckets = int(os.environ.get("DL4J_EXCHANGE_BUCKETS", "1"))
        if mode == "averaging" and buckets > 1 and hasattr(model, "tc") and model.flat_shadow is not None:
            # SameDiff training state with a low-precision shadow: exchange overlapped with backward, bucket by bucket
            from .fused import BucketedAveraging
            s = BucketedAveraging(fused, model, n_buckets=buckets)
            s.t, s.group, s.world, s.rank = t, group, fused.world, fused.rank
            s.broadcast_parameters = GradientSharing.broadcast_parameters.__get__(s)
        else:
            s = FusedAveraging(model, fused, group) if mode == "averaging" else FusedThresholdSharing(model, fused, thresholdAlgorithm, group)
    elif mode == "averaging":
        s = NcclAveraging(model, group)
    else:
        s = HostThresholdSharing(model, thresholdAlgorithm, residualPostProcessor, group)
    s.broadcast_parameters(0)
    model.gradient_hook = s
    return s


def _rehome(model, alloc):
    """Move the model's flat buffers into symmetric memory and rebuild every view of them."""
    if hasattr(model, "tc"):          # SameDiff TrainingState
        model.reallocate(alloc.empty)
    else:
        model._flat_allocator = alloc.empty
        dev = model.device
        p = alloc.empty(model.flat_params.numel(), model.flat_params.dtype, dev)
        p.copy_(model.flat_params)
        g = alloc.empty(model.flat_grads.numel(), model.flat_grads.dtype, dev)
        model.flat_params, model.flat_grads = p, g
        model._rebind()
