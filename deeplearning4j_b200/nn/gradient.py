"""``Gradient`` view object (``nn/gradient/DefaultGradient.java``): per-parameter views of the
flat gradient buffer keyed ``"<layer>_<param>"``."""
from __future__ import annotations

from ..nd.ndarray import INDArray
from .conf.base import flat_view


class Gradient:
    def __init__(self, net):
        self._net = net

    def gradient(self):
        return INDArray(self._net.flat_grads)

    def gradientForVariable(self):
        owners = self._net._owners()
        return {f"{owners[e.layer_index][0]}_{e.spec.name}": INDArray(flat_view(self._net.flat_grads, e.offset, e.spec))
                for e in self._net.entries}

    def getGradientFor(self, key):
        return self.gradientForVariable()[key]

    def clear(self):
        self._net.flat_grads.zero_()
