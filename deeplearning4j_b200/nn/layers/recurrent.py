"""Recurrent layers: LSTM, GravesLSTM (peepholes), SimpleRnn and the wrapper layers
Bidirectional / LastTimeStep / TimeDistributed.

Parameter layout follows ``nn/params/LSTMParamInitializer.java:118-193``:
``W('f',[nIn,4n]), RW('f',[n,4n]), b[1,4n]`` with gate blocks ``[i(block input), f, o, g]`` and
the forget-gate bias slice initialised to ``forgetGateBiasInit``; GravesLSTM's recurrent
matrix is ``[n, 4n+3]`` whose last three columns are the peephole weights
(``GravesLSTMParamInitializer.java``).  The time loop follows ``LSTMHelpers.java:66-330``:
one input GEMM for the whole sequence, then per step one recurrent GEMM and the fused cell.
State for truncated BPTT / ``rnnTimeStep`` is carried in ``ctx["rnn_state"]``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ...ops import nnops
from ..activations import Activation, ActivationSigmoid, ActivationTanH
from ..conf.base import BaseLayer, FeedForwardLayer, InputType, Layer, ParamSpec, RNNFormat, _L
from ..weights import WeightInit


class BaseRecurrentLayer(FeedForwardLayer):
    DEFAULTS = {"weightInitRecurrent": None, "rnnDataFormat": RNNFormat.NCW, "useBias": True}
    IS_RECURRENT = True

    def _finalise(self):
        super()._finalise()
        if self.weightInitRecurrent is not None:
            self.weightInitRecurrent = WeightInit.get(self.weightInitRecurrent)

    def setNIn(self, it, override):
        if not self.nIn or override:
            self.nIn = it.size

    def output_type(self, it):
        return InputType.recurrent(self.nOut, getattr(it, "timeSeriesLength", -1), self.rnnDataFormat)

    def preprocessor_for(self, it):
        from ..conf.preprocessors import FeedForwardToRnnPreProcessor, CnnToRnnPreProcessor
        if it.kind == InputType.FF:
            return FeedForwardToRnnPreProcessor(self.rnnDataFormat)
        if it.kind == InputType.CNN:
            return CnnToRnnPreProcessor(it.height, it.width, it.channels, self.rnnDataFormat)
        return None

    # [mb, n, T] <-> time-major [T, mb, n]
    def _to_tmn(self, x):
        return x.permute(2, 0, 1) if self.rnnDataFormat == RNNFormat.NCW else x.permute(1, 0, 2)

    def _from_tmn(self, y):
        return y.permute(1, 2, 0) if self.rnnDataFormat == RNNFormat.NCW else y.permute(1, 0, 2)

    def _state(self, ctx, key):
        if ctx is None:
            return None
        return ctx.get("rnn_state_in", {}).get(key)

    def _store(self, ctx, key, state):
        if ctx is not None:
            ctx.setdefault("rnn_state_out", {})[key] = state


class LSTM(BaseRecurrentLayer):
    JAVA_CLASS = _L + "LSTM"
    DEFAULTS = {"forgetGateBiasInit": 1.0, "gateActivationFn": None, "helperAllowFallback": True}
    PEEPHOLE = False

    def _finalise(self):
        super()._finalise()
        self.gateActivationFn = Activation.get(self.gateActivationFn or "SIGMOID")

    def resolved(self):
        super().resolved()
        if "activation" not in self._explicit and type(self.activation).__name__ == "ActivationSigmoid" and False:
            self.activation = Activation.get("TANH")
        return self

    def param_specs(self):
        n = self.nOut
        fg = self.forgetGateBiasInit

        def bias_init(out, gen):
            out.zero_()
            out.view(-1)[n:2 * n] = fg
        rw_cols = 4 * n + (3 if self.PEEPHOLE else 0)
        return [ParamSpec("W", (self.nIn, 4 * n), "f", "weight", self.nIn, n),
                ParamSpec("RW", (n, rw_cols), "f", "weight", n, n, init="recurrent"),
                ParamSpec("b", (1, 4 * n), "c", "bias", self.nIn, n, init=bias_init)]

    def forward(self, p, x, training, mask=None, ctx=None, reverse=False, key=None):
        x = self.apply_dropout(x, training)
        p = self.noisy(p, training)
        n = self.nOut
        xt = self._to_tmn(x)                                   # [T, mb, nIn]
        T, mb = xt.shape[0], xt.shape[1]
        key = key or id(self)
        st = self._state(ctx, key)
        if st is not None:
            h, c = st
        else:
            h = torch.zeros(mb, n, dtype=x.dtype, device=x.device)
            c = torch.zeros(mb, n, dtype=torch.float32 if x.dtype in (torch.bfloat16, torch.float16) else x.dtype, device=x.device)
        W, RW, b = p["W"], p["RW"], p["b"]
        RW4 = RW[:, :4 * n]
        # one GEMM for all time steps' input contributions
        zx = nnops.linear(xt.reshape(T * mb, -1), W, b).reshape(T, mb, 4 * n)
        gate, act = self.gateActivationFn, self.activation
        plain = isinstance(gate, ActivationSigmoid) and isinstance(act, ActivationTanH) and not self.PEEPHOLE
        if plain and mask is None and c.dtype == torch.float32 and not nnops._FORCE_TORCH:
            from ...ops import native as nat
            if nat.lstm_seq_supported(zx, n, mb) and h.dtype == zx.dtype:
                # whole sequence in one persistent kernel (recurrent weights resident on chip)
                hs, h, c = nat.lstm_seq(zx, RW if RW.shape[1] == 4 * n else RW4, h, c, reverse)
                self._store(ctx, key, (h, c))
                return self._from_tmn(hs)
        outs = [None] * T
        steps = range(T - 1, -1, -1) if reverse else range(T)
        mt = None if mask is None else mask.to(x.dtype).t().unsqueeze(2)   # [T, mb, 1]
        for t in steps:
            z = zx[t] + nnops.linear(h, RW4, None)
            if plain:
                h_new, c_new = nnops.lstm_cell(z, c)
            else:
                a = act(z[:, :n])
                zf, zo, zg = z[:, n:2 * n], z[:, 2 * n:3 * n], z[:, 3 * n:]
                if self.PEEPHOLE:
                    zf = zf + c.to(z.dtype) * RW[:, 4 * n].to(z.dtype)
                    zg = zg + c.to(z.dtype) * RW[:, 4 * n + 2].to(z.dtype)
                f, g = gate(zf), gate(zg)
                c_new = f * c.to(z.dtype) + g * a
                if self.PEEPHOLE:
                    zo = zo + c_new * RW[:, 4 * n + 1].to(z.dtype)
                o = gate(zo)
                h_new = o * act(c_new)
                c_new = c_new.to(c.dtype)
            if mt is not None:
                m = mt[t]
                h_new = m * h_new + (1 - m) * h
                c_new = (m * c_new.to(x.dtype) + (1 - m) * c.to(x.dtype)).to(c.dtype)
                outs[t] = h_new * m
            else:
                outs[t] = h_new
            h, c = h_new.to(x.dtype), c_new
        self._store(ctx, key, (h, c))
        return self._from_tmn(torch.stack(outs, 0))


class GravesLSTM(LSTM):
    JAVA_CLASS = _L + "GravesLSTM"
    PEEPHOLE = True


class SimpleRnn(BaseRecurrentLayer):
    """``h_t = act(x_t W + h_{t-1} RW + b)`` with optional layer norm (``SimpleRnn.java``)."""
    JAVA_CLASS = _L + "recurrent.SimpleRnn"
    DEFAULTS = {"hasLayerNorm": False}

    def param_specs(self):
        n = self.nOut
        s = [ParamSpec("W", (self.nIn, n), "f", "weight", self.nIn, n),
             ParamSpec("RW", (n, n), "f", "weight", n, n, init="recurrent"),
             ParamSpec("b", (1, n), "c", "bias", self.nIn, n)]
        if self.hasLayerNorm:
            s.append(ParamSpec("g", (1, 2 * n), "c", "gain", n, n))
        return s

    def forward(self, p, x, training, mask=None, ctx=None, reverse=False, key=None):
        x = self.apply_dropout(x, training)
        n = self.nOut
        xt = self._to_tmn(x)
        T, mb = xt.shape[0], xt.shape[1]
        key = key or id(self)
        st = self._state(ctx, key)
        h = st[0] if st is not None else torch.zeros(mb, n, dtype=x.dtype, device=x.device)
        zx = nnops.linear(xt.reshape(T * mb, -1), p["W"], None).reshape(T, mb, n)
        if self.hasLayerNorm:
            g = p["g"].reshape(-1)
            zx = F.layer_norm(zx, (n,), g[:n].to(zx.dtype), None, 1e-5)
        outs = [None] * T
        mt = None if mask is None else mask.to(x.dtype).t().unsqueeze(2)
        for t in (range(T - 1, -1, -1) if reverse else range(T)):
            r = nnops.linear(h, p["RW"], None)
            if self.hasLayerNorm:
                r = F.layer_norm(r, (n,), g[n:].to(r.dtype), None, 1e-5)
            h_new = self.activation(zx[t] + r + p["b"].to(zx.dtype), training)
            if mt is not None:
                h_new = mt[t] * h_new + (1 - mt[t]) * h
                outs[t] = h_new * mt[t]
            else:
                outs[t] = h_new
            h = h_new
        self._store(ctx, key, (h,))
        return self._from_tmn(torch.stack(outs, 0))


class _Wrapper(Layer):
    DEFAULTS = {"underlying": None}

    def _positional(self, *args):
        if args:
            self.underlying = args[-1]
            if len(args) == 2:
                self.mode = args[0]

    @property
    def HAS_PARAMS(self):
        return self.underlying.HAS_PARAMS

    def apply_global(self, g): self.underlying.apply_global(g)
    def resolved(self):
        if hasattr(self.underlying, "resolved"):
            self.underlying.resolved()
        return self
    def setNIn(self, it, o): self.underlying.setNIn(it, o)
    def output_type(self, it): return self.underlying.output_type(it)
    def preprocessor_for(self, it): return self.underlying.preprocessor_for(it)
    def param_specs(self): return self.underlying.param_specs()
    def regularizers(self, s): return self.underlying.regularizers(s)
    def updater_for(self, s): return self.underlying.updater_for(s)

    @property
    def nIn(self): return self.underlying.nIn
    @property
    def nOut(self): return self.underlying.nOut
    @property
    def activation(self): return getattr(self.underlying, "activation", None)

    def to_json(self):
        d = {"@class": self.JAVA_CLASS, "underlying": self.underlying.to_json()}
        return d


class Bidirectional(_Wrapper):
    """Runs two copies of a recurrent layer (forward / time-reversed) and combines them.
    Parameters are the forward copy's followed by the backward copy's, prefixed ``f`` / ``b``
    (``BidirectionalParamInitializer.java``)."""
    JAVA_CLASS = _L + "recurrent.Bidirectional"
    DEFAULTS = {"mode": "CONCAT", "fwd": None, "bwd": None}
    IS_RECURRENT = True

    class Mode:
        ADD = "ADD"; MUL = "MUL"; AVERAGE = "AVERAGE"; CONCAT = "CONCAT"

    def _finalise(self):
        super()._finalise()
        if self.underlying is not None and self.fwd is None:
            self.fwd = self.underlying
            self.bwd = self.underlying.clone()

    def apply_global(self, g):
        self.fwd.apply_global(g); self.bwd.apply_global(g)

    def resolved(self):
        self.fwd.resolved(); self.bwd.resolved(); return self

    def setNIn(self, it, o):
        self.fwd.setNIn(it, o); self.bwd.setNIn(it, o)

    @property
    def nOut(self):
        return self.fwd.nOut * (2 if self.mode == "CONCAT" else 1)

    @property
    def nIn(self):
        return self.fwd.nIn

    def output_type(self, it):
        o = self.fwd.output_type(it)
        return InputType.recurrent(self.nOut, o.timeSeriesLength, o.format)

    def param_specs(self):
        out = []
        for pre, l in (("f", self.fwd), ("b", self.bwd)):
            for s in l.param_specs():
                out.append(ParamSpec(pre + s.name, s.shape, s.order, s.kind, s.fanIn, s.fanOut, s.init))
        return out

    def regularizers(self, spec):
        return self.fwd.regularizers(ParamSpec(spec.name[1:], spec.shape, spec.order, spec.kind))

    def updater_for(self, spec):
        return self.fwd.updater_for(ParamSpec(spec.name[1:], spec.shape, spec.order, spec.kind))

    def forward(self, p, x, training, mask=None, ctx=None):
        pf = {k[1:]: v for k, v in p.items() if k.startswith("f")}
        pb = {k[1:]: v for k, v in p.items() if k.startswith("b")}
        yf = self.fwd.forward(pf, x, training, mask, ctx, reverse=False, key=(id(self), "f"))
        yb = self.bwd.forward(pb, x, training, mask, ctx, reverse=True, key=(id(self), "b"))
        if self.mode == "ADD":
            return yf + yb
        if self.mode == "MUL":
            return yf * yb
        if self.mode == "AVERAGE":
            return 0.5 * (yf + yb)
        return torch.cat([yf, yb], dim=1 if self.fwd.rnnDataFormat == RNNFormat.NCW else 2)

    def to_json(self):
        return {"@class": self.JAVA_CLASS, "bwd": self.bwd.to_json(), "fwd": self.fwd.to_json(), "mode": self.mode}


class LastTimeStep(_Wrapper):
    """Returns the activations of the last (unmasked) time step: [mb, n, T] -> [mb, n]."""
    JAVA_CLASS = _L + "recurrent.LastTimeStep"

    def output_type(self, it):
        o = self.underlying.output_type(it)
        return InputType.feedForward(o.size)

    def forward(self, p, x, training, mask=None, ctx=None):
        y = self.underlying.forward(p, x, training, mask, ctx)
        if getattr(self.underlying, "rnnDataFormat", RNNFormat.NCW) == RNNFormat.NWC:
            y = y.permute(0, 2, 1)
        if mask is None:
            return y[:, :, -1]
        T = y.shape[2]
        idx = (mask.to(torch.long) * torch.arange(T, device=y.device)).argmax(dim=1)
        return y.gather(2, idx.reshape(-1, 1, 1).expand(-1, y.shape[1], 1)).squeeze(2)

    def feed_forward_mask(self, mask, input_type=None):
        return None


class TimeDistributed(_Wrapper):
    """Applies a feed-forward layer independently at every time step."""
    JAVA_CLASS = _L + "recurrent.TimeDistributed"
    DEFAULTS = {"rnnDataFormat": RNNFormat.NCW}

    def setNIn(self, it, o):
        self.underlying.setNIn(InputType.feedForward(it.size) if it.kind == InputType.RNN else it, o)

    def output_type(self, it):
        o = self.underlying.output_type(InputType.feedForward(it.size))
        return InputType.recurrent(o.size, it.timeSeriesLength, self.rnnDataFormat)

    def preprocessor_for(self, it):
        return None

    def forward(self, p, x, training, mask=None, ctx=None):
        ncw = self.rnnDataFormat == RNNFormat.NCW
        xt = x.permute(0, 2, 1) if ncw else x
        mb, T = xt.shape[0], xt.shape[1]
        y = self.underlying.forward(p, xt.reshape(mb * T, -1), training, None, ctx).reshape(mb, T, -1)
        return y.permute(0, 2, 1) if ncw else y

    def to_json(self):
        return {"@class": self.JAVA_CLASS, "rnnDataFormat": self.rnnDataFormat, "underlying": self.underlying.to_json()}
