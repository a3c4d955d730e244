"""Attention layers (``SelfAttentionLayer``, ``LearnedSelfAttentionLayer``,
``RecurrentAttentionLayer``, ``DotProductAttentionLayer``).

The reference builds these as SameDiff layers around ``multi_head_dot_product_attention``
(``nn/conf/layers/SelfAttentionLayer.java``; native op
``libnd4j/include/ops/declarable/generic/nn/multi_head_dot_product_attention.cpp:99-134``).
Parameters: ``Wq, Wk, Wv`` as ``[nHeads, headSize, nIn]`` and ``Wo`` as
``[nHeads*headSize, nOut]``; without projection the input is used directly (nHeads must be 1).
Activations are [mb, n, T]; the score matrix is never materialised on the fused CUDA path.
"""
from __future__ import annotations

import math

import torch

from ...ops import nnops
from ..conf.base import BaseLayer, FeedForwardLayer, InputType, ParamSpec, RNNFormat, _L


def _mha(x_q, x_kv, p, n_heads, head, project, mask, training):
    """x_q [mb, nIn, Tq], x_kv [mb, nIn, Tk] -> [mb, nOut, Tq]."""
    if not project:
        q = x_q.permute(0, 2, 1).unsqueeze(1)
        k = v = x_kv.permute(0, 2, 1).unsqueeze(1)
        o = nnops.attention(q, k, v, mask)
        return o.squeeze(1).permute(0, 2, 1)
    mb, _, tq = x_q.shape
    tk = x_kv.shape[2]
    def proj(x, W):   # W [h, d, nIn]
        Wf = W.reshape(n_heads * head, -1).t()                      # [nIn, h*d]
        y = nnops.linear(x.permute(0, 2, 1).reshape(-1, x.shape[1]), Wf.to(x.dtype), None)
        return y.reshape(x.shape[0], -1, n_heads, head).permute(0, 2, 1, 3)   # [mb, h, T, d]
    q, k, v = proj(x_q, p["Wq"]), proj(x_kv, p["Wk"]), proj(x_kv, p["Wv"])
    o = nnops.attention(q, k, v, mask)                               # [mb, h, Tq, d]
    o = o.permute(0, 2, 1, 3).reshape(mb * tq, n_heads * head)
    y = nnops.linear(o, p["Wo"].to(o.dtype), None)
    return y.reshape(mb, tq, -1).permute(0, 2, 1)


class SelfAttentionLayer(FeedForwardLayer):
    JAVA_CLASS = _L + "SelfAttentionLayer"
    DEFAULTS = {"nHeads": 1, "headSize": 0, "projectInput": False}

    def _finalise(self):
        super()._finalise()
        if self.projectInput and not self.headSize and self.nOut:
            self.headSize = self.nOut // self.nHeads

    def setNIn(self, it, override):
        if not self.nIn or override:
            self.nIn = it.size
        if not self.projectInput:
            self.nOut = self.nIn

    def output_type(self, it):
        return InputType.recurrent(self.nOut, it.timeSeriesLength, getattr(it, "format", RNNFormat.NCW))

    def preprocessor_for(self, it):
        return None

    def param_specs(self):
        if not self.projectInput:
            return []
        h, d = self.nHeads, self.headSize
        return [ParamSpec("Wq", (h, d, self.nIn), "c", "weight", self.nIn, d),
                ParamSpec("Wk", (h, d, self.nIn), "c", "weight", self.nIn, d),
                ParamSpec("Wv", (h, d, self.nIn), "c", "weight", self.nIn, d),
                ParamSpec("Wo", (h * d, self.nOut), "c", "weight", h * d, self.nOut)]

    def forward(self, p, x, training, mask=None, ctx=None):
        return _mha(x, x, p, self.nHeads, self.headSize, self.projectInput, mask, training)


class LearnedSelfAttentionLayer(SelfAttentionLayer):
    """Attention with ``nQueries`` learned query vectors: output [mb, nOut, nQueries]."""
    JAVA_CLASS = _L + "LearnedSelfAttentionLayer"
    DEFAULTS = {"nQueries": 1}

    def output_type(self, it):
        return InputType.recurrent(self.nOut, self.nQueries, getattr(it, "format", RNNFormat.NCW))

    def param_specs(self):
        s = super().param_specs()
        s.append(ParamSpec("Q", (1, self.nIn, self.nQueries), "c", "weight", self.nIn, self.nQueries))
        return s

    def forward(self, p, x, training, mask=None, ctx=None):
        q = p["Q"].to(x.dtype).expand(x.shape[0], -1, -1)
        return _mha(q, x, p, self.nHeads, self.headSize, self.projectInput, mask, training)

    def feed_forward_mask(self, mask, input_type=None):
        return None


class RecurrentAttentionLayer(FeedForwardLayer):
    """``h_t = act(x_t W + attention(h_{t-1}; x) RW + b)`` (``RecurrentAttentionLayer.java``)."""
    JAVA_CLASS = _L + "RecurrentAttentionLayer"
    DEFAULTS = {"nHeads": 1, "headSize": 0, "projectInput": True, "hasBias": True}

    def _finalise(self):
        super()._finalise()
        if not self.headSize and self.nOut:
            self.headSize = self.nOut // self.nHeads

    def setNIn(self, it, override):
        if not self.nIn or override:
            self.nIn = it.size

    def output_type(self, it):
        return InputType.recurrent(self.nOut, it.timeSeriesLength, getattr(it, "format", RNNFormat.NCW))

    def preprocessor_for(self, it):
        return None

    def param_specs(self):
        h, d, n = self.nHeads, self.headSize, self.nOut
        s = [ParamSpec("W", (self.nIn, n), "c", "weight", self.nIn, n),
             ParamSpec("RW", (n, n), "c", "weight", n, n)]
        if self.hasBias:
            s.append(ParamSpec("b", (1, n), "c", "bias", self.nIn, n))
        if self.projectInput:
            s += [ParamSpec("Wq", (h, d, n), "c", "weight", n, d), ParamSpec("Wk", (h, d, self.nIn), "c", "weight", self.nIn, d),
                  ParamSpec("Wv", (h, d, self.nIn), "c", "weight", self.nIn, d), ParamSpec("Wo", (h * d, n), "c", "weight", h * d, n)]
        return s

    def forward(self, p, x, training, mask=None, ctx=None):
        mb, _, T = x.shape
        n = self.nOut
        zx = nnops.linear(x.permute(0, 2, 1).reshape(mb * T, -1), p["W"].to(x.dtype), p.get("b")).reshape(mb, T, n)
        h = torch.zeros(mb, n, dtype=x.dtype, device=x.device)
        outs = []
        for t in range(T):
            a = _mha(h.unsqueeze(2), x, p, self.nHeads, self.headSize, self.projectInput, mask, training).squeeze(2)
            h = self.activation(zx[:, t] + a @ p["RW"].to(x.dtype), training)
            outs.append(h)
        return torch.stack(outs, 2)


class DotProductAttentionLayer(BaseLayer):
    """Parameter-free scaled dot-product attention over a [queries, keys, values] triple packed
    by the caller; used through ``DotProductAttentionVertex`` in graphs."""
    JAVA_CLASS = _L + "DotProductAttentionLayer"
    DEFAULTS = {"scaleFactor": None, "dropoutProbability": 0.0, "useCausalMask": False, "training": False, "nIn": 0, "nOut": 0}
    HAS_PARAMS = False

    def setNIn(self, it, override):
        self.nIn = self.nOut = it.size

    def output_type(self, it):
        return it

    def forward(self, p, x, training, mask=None, ctx=None):
        q = k = v = x.permute(0, 2, 1).unsqueeze(1)
        if self.useCausalMask:
            T = q.shape[2]
            causal = torch.full((T, T), float("-inf"), device=x.device, dtype=torch.float32).triu(1)
            o = nnops.attention(q, k, v, causal[None, None], self.scaleFactor, self.dropoutProbability, training)
        else:
            o = nnops.attention(q, k, v, mask, self.scaleFactor, self.dropoutProbability, training)
        return o.squeeze(1).permute(0, 2, 1)
