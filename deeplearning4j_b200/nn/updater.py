"""Network-level updater: ``BaseMultiLayerUpdater`` + ``UpdaterBlock``.

Parity: ``deeplearning4j-nn/.../nn/updater/BaseMultiLayerUpdater.java:65-180`` (block
construction: consecutive parameters whose updater configurations are equal share one block
and one contiguous slice of the state view), ``:261-315`` (update order: gradient
normalisation -> per block regularisation -> updater -> weight decay) and
``UpdaterBlock.java:118-165``.

The flat state view is the concatenation of the blocks' states in parameter order, which is
what ``updaterState.bin`` stores.  On CUDA the whole update (regularisation, updater math,
``params -= update`` and zeroing the gradient for the next iteration) is one launch of the
multi-segment kernel in ``ops.native``; the torch path below is the oracle / CPU path.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from .conf.base import GradientNormalization
from .updaters import (GradientUpdater, IUpdater, L1Regularization, L2Regularization, Nesterovs, NoOp, Sgd,
                       WeightDecay, ISchedule)


@dataclass
class ParamEntry:
    layer_index: int          # index into the owner's layer list (or vertex order)
    layer: object
    spec: object
    offset: int               # into the flat params / gradient buffers
    key: str                  # "<layerIdx or vertexName>_<paramName>"

    @property
    def end(self):
        return self.offset + self.spec.numel


@dataclass
class UpdaterBlock:
    config: IUpdater
    entries: list = field(default_factory=list)
    state_offset: int = 0

    @property
    def start(self):
        return self.entries[0].offset

    @property
    def end(self):
        return self.entries[-1].end

    @property
    def numel(self):
        return self.end - self.start

    @property
    def state_size(self):
        return self.config.stateSize(self.numel)


def _lr_key(u: IUpdater):
    return u.to_json() if u is not None else None


def build_blocks(entries):
    blocks = []
    for e in entries:
        u = e.layer.updater_for(e.spec) if hasattr(e.layer, "updater_for") else None
        if u is None:
            u = NoOp()
        if blocks and blocks[-1].config == u and blocks[-1].end == e.offset:
            blocks[-1].entries.append(e)
        else:
            blocks.append(UpdaterBlock(u, [e]))
    off = 0
    for b in blocks:
        b.state_offset = off
        off += b.state_size
    return blocks, off


class MultiLayerUpdater:
    def __init__(self, entries, params_flat: torch.Tensor, grads_flat: torch.Tensor, state_view=None):
        self.entries = entries
        self.params = params_flat
        self.grads = grads_flat
        self.blocks, self.state_size = build_blocks(entries)
        if state_view is None:
            state_view = torch.zeros(self.state_size, dtype=params_flat.dtype, device=params_flat.device)
        self.state = state_view
        self._bind()
        self._seg_table = None
        self.shadow = None            # optional low-precision parameter shadow refreshed by the fused kernel
        self.shadow_offsets = None
        self._shadow_fresh = False

    def _bind(self):
        self.updaters = []
        for b in self.blocks:
            sv = self.state[b.state_offset:b.state_offset + b.state_size]
            self.updaters.append(GradientUpdater(b.config, sv, initialize=False))

    # ------------------------------------------------------------------ state view
    def getStateViewArray(self):
        return self.state

    def setStateViewArray(self, view):
        if view is None:
            return
        v = view.reshape(-1)
        if v.numel() != self.state_size:
            raise ValueError(f"updater state length {v.numel()} != expected {self.state_size}")
        self.state.copy_(v.to(self.state.dtype).to(self.state.device))

    # ------------------------------------------------------------------ update
    def _pre_apply(self):
        """Gradient normalisation / clipping per layer (``BaseMultiLayerUpdater.preApply``)."""
        by_layer = {}
        for e in self.entries:
            by_layer.setdefault(e.layer_index, []).append(e)
        for es in by_layer.values():
            layer = es[0].layer
            gn = getattr(layer, "gradientNormalization", None)
            if gn in (None, GradientNormalization.None_):
                continue
            thr = getattr(layer, "gradientNormalizationThreshold", 1.0) or 1.0
            views = [self.grads[e.offset:e.end] for e in es if e.spec.kind != "state"]
            if not views:
                continue
            if gn == GradientNormalization.RenormalizeL2PerLayer:
                n = math.sqrt(sum(float((v * v).sum()) for v in views))
                if n > 0:
                    for v in views:
                        v.div_(n)
            elif gn == GradientNormalization.RenormalizeL2PerParamType:
                for v in views:
                    n = float(v.norm(2))
                    if n > 0:
                        v.div_(n)
            elif gn == GradientNormalization.ClipElementWiseAbsoluteValue:
                for v in views:
                    v.clamp_(-thr, thr)
            elif gn == GradientNormalization.ClipL2PerLayer:
                n = math.sqrt(sum(float((v * v).sum()) for v in views))
                if n > thr:
                    for v in views:
                        v.mul_(thr / n)
            elif gn == GradientNormalization.ClipL2PerParamType:
                for v in views:
                    n = float(v.norm(2))
                    if n > thr:
                        v.mul_(thr / n)

    def needs_pre_apply(self):
        return any(getattr(e.layer, "gradientNormalization", None) not in (None, GradientNormalization.None_)
                   for e in self.entries)

    def update(self, iteration: int, epoch: int, apply_step: bool = True, use_fused: bool | None = None):
        """Turn ``grads`` into the update and (if ``apply_step``) do ``params -= update``."""
        if self.needs_pre_apply():
            self._pre_apply()
        if use_fused is None:
            from ..ops import nnops
            use_fused = self.params.is_cuda and not nnops._FORCE_TORCH        # the library-only baseline also updates with torch ops
        self._shadow_fresh = False
        if use_fused and apply_step and self._fused_update(iteration, epoch):
            self._shadow_fresh = self.shadow is not None
            return
        for b, gu in zip(self.blocks, self.updaters):
            cfg = b.config
            lr = cfg.getLearningRate(iteration, epoch) if cfg.hasLearningRate() else 0.0
            for e in b.entries:
                if e.spec.kind == "state":
                    continue
                g = self.grads[e.offset:e.end]
                p = self.params[e.offset:e.end]
                for r in e.layer.regularizers(e.spec):
                    if r.APPLY_STEP == "BEFORE_UPDATER":
                        r.apply(p, g, lr, iteration, epoch)
            g_block = self.grads[b.start:b.end]
            if not isinstance(cfg, NoOp):
                gu.applyUpdater(g_block, iteration, epoch)
            else:
                g_block.zero_()
            for e in b.entries:
                if e.spec.kind == "state":
                    continue
                for r in e.layer.regularizers(e.spec):
                    if r.APPLY_STEP == "POST_UPDATER":
                        r.apply(self.params[e.offset:e.end], self.grads[e.offset:e.end], lr, iteration, epoch)
        if apply_step:
            self.params.sub_(self.grads)

    # ------------------------------------------------------------------ fused CUDA path
    def segments(self, iteration, epoch):
        """Per-parameter segment list for the fused kernel:
        (offset, numel, state_offset_of_block, block_numel, block_start, kernel_id, lr, l1, l2, wd, hyper...)."""
        segs = []
        for b in self.blocks:
            cfg = b.config
            lr = cfg.getLearningRate(iteration, epoch) if cfg.hasLearningRate() else 0.0
            for e in b.entries:
                l1 = l2 = wd = 0.0
                if e.spec.kind != "state":
                    for r in e.layer.regularizers(e.spec):
                        v = r.value(iteration, epoch)
                        if isinstance(r, L1Regularization):
                            l1 += v
                        elif isinstance(r, L2Regularization):
                            l2 += v
                        elif isinstance(r, WeightDecay):
                            wd += v * (lr if r.applyLR else 1.0)
                kid = 9 if e.spec.kind == "state" else cfg.KERNEL_ID
                segs.append((e.offset, e.spec.numel, b.state_offset, b.numel, b.start, kid, lr, l1, l2, wd, cfg))
        return segs

    def _fused_update(self, iteration, epoch) -> bool:
        from ..ops import native
        if not native.available() or self.params.dtype != torch.float32:
            return False
        return native.fused_update(self, iteration, epoch, self.shadow, self.shadow_offsets)
