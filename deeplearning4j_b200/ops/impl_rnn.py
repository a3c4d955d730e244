"""Recurrent ops (``headers/recurrent.h``): lstmLayer / lstmLayerCell / lstmCell / lstmBlock(Cell),
gru / gruCell, sru / sruCell / sru_bi, static / dynamic (bidirectional) rnn.

Gate order of the ``lstmLayer`` family is [i, f, c(g), o] with weights ``Wx [nIn, 4n]``,
``Wr [n, 4n]``, ``b [4n]`` and optional peepholes ``Wp [3n]``
(``libnd4j/include/ops/declarable/helpers/impl/lstmLayer.cpp``).  The time loop does one input GEMM
for all steps and one recurrent GEMM per step through ``nnops.linear`` (tcgen05 on a B200)."""
from __future__ import annotations

import torch

from . import nnops
from .registry import op
from .impl_nn import _autobp

_ACTS = [torch.tanh, torch.relu, torch.sigmoid, lambda x: x, lambda x: torch.nn.functional.leaky_relu(x, 0.01),
         lambda x: torch.clamp(x, 0, 1), torch.nn.functional.elu, torch.nn.functional.softsign,
         torch.nn.functional.hardsigmoid, torch.nn.functional.hardtanh, torch.nn.functional.softplus]


def _act(i, default):
    return _ACTS[int(i)] if i is not None else default


def _lstm_step(zx, h, c, Wr, Wp, n, gate, cell, out, clip=0.0):
    z = zx + nnops.linear(h, Wr, None)
    zi, zf, zc, zo = z[:, :n], z[:, n:2 * n], z[:, 2 * n:3 * n], z[:, 3 * n:]
    if Wp is not None:
        zi = zi + c * Wp[:n]
        zf = zf + c * Wp[n:2 * n]
    i, f = gate(zi), gate(zf)
    cn = f * c + i * cell(zc)
    if clip:
        cn = cn.clamp(-clip, clip)
    if Wp is not None:
        zo = zo + cn * Wp[2 * n:]
    o = gate(zo)
    return o * out(cn), cn


@op("lstmLayer", n_out=-1)
def lstmLayer(x, Wx, Wr, b=None, seqLen=None, hI=None, cI=None, Wp=None, dataFormat=0, directionMode=0, gateAct=2, cellAct=0,
              outAct=0, retFullSeq=True, retLastH=False, retLastC=False, cellClip=0.0, **kw):
    """dataFormat: 0 = [T, B, nIn], 1 = [B, T, nIn], 2 = [B, nIn, T]; directionMode: 0 fwd, 1 bwd,
    2 bidirectional sum, 3 bidirectional concat."""
    df = int(dataFormat)
    xt = x if df == 0 else (x.permute(1, 0, 2) if df == 1 else x.permute(2, 0, 1))
    T, B, _ = xt.shape
    dm = int(directionMode)
    gate, cell, out = _act(gateAct, torch.sigmoid), _act(cellAct, torch.tanh), _act(outAct, torch.tanh)

    def run(direction, Wx_, Wr_, b_, Wp_, h0, c0):
        n = Wr_.shape[0]
        h = h0 if h0 is not None else torch.zeros(B, n, dtype=x.dtype, device=x.device)
        c = c0 if c0 is not None else torch.zeros(B, n, dtype=x.dtype, device=x.device)
        zx = nnops.linear(xt.reshape(T * B, -1), Wx_, b_).reshape(T, B, 4 * n)
        hs = [None] * T
        for t in (range(T - 1, -1, -1) if direction else range(T)):
            hn, cn = _lstm_step(zx[t], h, c, Wr_, Wp_, n, gate, cell, out, cellClip)
            if seqLen is not None:
                m = (t < seqLen).to(x.dtype).unsqueeze(1)
                hn, cn = m * hn + (1 - m) * h, m * cn + (1 - m) * c
                hs[t] = hn * m
            else:
                hs[t] = hn
            h, c = hn, cn
        return torch.stack(hs, 0), h, c
    if dm in (0, 1):
        hseq, hL, cL = run(dm, Wx, Wr, b, Wp, hI, cI)
    else:
        f = run(0, Wx[0], Wr[0], None if b is None else b[0], None if Wp is None else Wp[0],
                None if hI is None else hI[0], None if cI is None else cI[0])
        r = run(1, Wx[1], Wr[1], None if b is None else b[1], None if Wp is None else Wp[1],
                None if hI is None else hI[1], None if cI is None else cI[1])
        if dm == 2:
            hseq = f[0] + r[0]
        else:
            hseq = torch.cat([f[0], r[0]], -1)
        hL, cL = torch.stack([f[1], r[1]]), torch.stack([f[2], r[2]])
    outs = []
    if retFullSeq:
        outs.append(hseq if df == 0 else (hseq.permute(1, 0, 2) if df == 1 else hseq.permute(1, 2, 0)))
    if retLastH:
        outs.append(hL)
    if retLastC:
        outs.append(cL)
    return tuple(outs)


op("lstmLayer_bp", n_out=-1)(_autobp(lambda *a, **kw: lstmLayer(*a, **kw)[0], 4))


@op("lstmLayerCell", n_out=2)
def lstmLayerCell(x, Wx, Wr, b=None, hI=None, cI=None, Wp=None, gateAct=2, cellAct=0, outAct=0, cellClip=0.0, **kw):
    n = Wr.shape[0]
    h = hI if hI is not None else torch.zeros(x.shape[0], n, dtype=x.dtype, device=x.device)
    c = cI if cI is not None else torch.zeros_like(h)
    return _lstm_step(nnops.linear(x, Wx, b), h, c, Wr, Wp, n, _act(gateAct, torch.sigmoid), _act(cellAct, torch.tanh),
                      _act(outAct, torch.tanh), cellClip)


op("lstmLayerCellBp", n_out=-1)(_autobp(lambda *a, **kw: lstmLayerCell(*a, **kw)[0], 3))


@op("lstmCell", n_out=2)
def lstmCell(xt, ht_1, ct_1, Wx, Wh, Wc, Wp, b, peephole=False, projection=False, clippingCellValue=0.0, clippingProjValue=0.0,
             forgetBias=0.0, **kw):
    """Legacy cell: gate order [i, c, f, o] with z = x Wx + h Wh + b (``helpers/cuda/lstm.cu:45-110``)."""
    n = ct_1.shape[1]
    z = xt @ Wx + ht_1 @ Wh + b
    zi, zc, zf, zo = z[:, :n], z[:, n:2 * n], z[:, 2 * n:3 * n], z[:, 3 * n:]
    if peephole:
        zi = zi + ct_1 * Wc[:n]
        zf = zf + ct_1 * Wc[n:2 * n]
    i, f = torch.sigmoid(zi), torch.sigmoid(zf + forgetBias)
    c = f * ct_1 + i * torch.tanh(zc)
    if clippingCellValue:
        c = c.clamp(-clippingCellValue, clippingCellValue)
    if peephole:
        zo = zo + c * Wc[2 * n:]
    h = torch.sigmoid(zo) * torch.tanh(c)
    if projection:
        h = h @ Wp
        if clippingProjValue:
            h = h.clamp(-clippingProjValue, clippingProjValue)
    return h, c


@op("lstmBlockCell", n_out=7)
def lstmBlockCell(xt, cLast, yLast, W, Wci, Wcf, Wco, b, peephole=False, forgetBias=0.0, clippingCellValue=0.0, **kw):
    """TF ``LSTMBlockCell``: W [(nIn+n), 4n], gate order [i, c(g), f, o]; returns (i, c, f, o, z, h, y)."""
    n = cLast.shape[1]
    z = torch.cat([xt, yLast], 1) @ W + b
    zi, zg, zf, zo = z[:, :n], z[:, n:2 * n], z[:, 2 * n:3 * n], z[:, 3 * n:]
    if peephole:
        zi, zf = zi + cLast * Wci, zf + cLast * Wcf
    i, g, f = torch.sigmoid(zi), torch.tanh(zg), torch.sigmoid(zf + forgetBias)
    c = f * cLast + i * g
    if clippingCellValue:
        c = c.clamp(-clippingCellValue, clippingCellValue)
    if peephole:
        zo = zo + c * Wco
    o = torch.sigmoid(zo)
    hh = torch.tanh(c)
    return i, c, f, o, g, hh, o * hh


@op("lstmBlock", n_out=7)
def lstmBlock(maxTSLength, x, cLast, yLast, W, Wci, Wcf, Wco, b, peephole=False, forgetBias=0.0, clippingCellValue=0.0,
              dataFormat=0, **kw):
    df = int(dataFormat)
    xt = x if df == 0 else (x.permute(2, 0, 1) if df == 1 else x.permute(1, 0, 2))
    outs = [[] for _ in range(7)]
    c, y = cLast, yLast
    for t in range(xt.shape[0]):
        r = lstmBlockCell(xt[t], c, y, W, Wci, Wcf, Wco, b, peephole, forgetBias, clippingCellValue)
        for o, v in zip(outs, r):
            o.append(v)
        c, y = r[1], r[6]

    def fmt(s):
        s = torch.stack(s, 0)
        return s if df == 0 else (s.permute(1, 2, 0) if df == 1 else s.permute(1, 0, 2))
    return tuple(fmt(o) for o in outs)


@op("lstm", n_out=2)
def lstm(x, h0, c0, Wx, Wh, Wc, Wp, b, **kw):
    hs, h, c = [], h0, c0
    for t in range(x.shape[0]):
        h, c = lstmCell(x[t], h, c, Wx, Wh, Wc, Wp, b, **kw)
        hs.append(h)
    return torch.stack(hs, 0), c


@op("gruCell", n_out=4)
def gruCell(x, hLast, Wru, Wc, bru, bc, **kw):
    """Wru [(nIn+n), 2n] (reset | update), Wc [(nIn+n), n]; returns (r, u, c, h)."""
    n = hLast.shape[1]
    ru = torch.sigmoid(torch.cat([x, hLast], 1) @ Wru + bru)
    r, u = ru[:, :n], ru[:, n:]
    c = torch.tanh(torch.cat([x, r * hLast], 1) @ Wc + bc)
    return r, u, c, u * hLast + (1 - u) * c


@op("gruCell_bp", n_out=6)
def gruCell_bp(x, hLast, Wru, Wc, bru, bc, dLdr, dLdu=None, dLdc=None, dLdh=None, **kw):
    """Gradients of (x, hLast, Wru, Wc, bru, bc) given the gradients of the four outputs (r, u, c, h), in the reference's input
    order (``generic/nn/recurrent/gruCell.cpp:134-150``); with one gradient only it is taken as dL/dh."""
    if dLdu is None and dLdc is None and dLdh is None:
        dLdr, dLdh = None, dLdr
    with torch.enable_grad():
        leaves = [t.detach().clone().requires_grad_(True) for t in (x, hLast, Wru, Wc, bru, bc)]
        outs = gruCell(*leaves)
        pairs = [(o, g) for o, g in zip(outs, (dLdr, dLdu, dLdc, dLdh)) if g is not None]
        grads = torch.autograd.grad([o for o, _ in pairs], leaves, [g for _, g in pairs], allow_unused=True)
    return tuple(torch.zeros_like(l) if g is None else g for l, g in zip(leaves, grads))


@op("gru")
def gru(x, hI, Wx, Wh, b, **kw):
    """x [T, B, nIn]; Wx [nIn, 3n], Wh [n, 3n] with gate order [r, u, c]; b [3n] (``helpers/impl/gru.cpp``)."""
    n = hI.shape[1]
    T, B, _ = x.shape
    zx = nnops.linear(x.reshape(T * B, -1), Wx, b).reshape(T, B, 3 * n)
    h, hs = hI, []
    for t in range(T):
        zh = nnops.linear(h, Wh, None)
        r = torch.sigmoid(zx[t][:, :n] + zh[:, :n])
        u = torch.sigmoid(zx[t][:, n:2 * n] + zh[:, n:2 * n])
        c = torch.tanh(zx[t][:, 2 * n:] + r * zh[:, 2 * n:])
        h = u * h + (1 - u) * c
        hs.append(h)
    return torch.stack(hs, 0)


op("gru_bp", n_out=-1)(_autobp(gru, 5))


@op("sruCell", n_out=2)
def sruCell(xt, ct_1, W, b, **kw):
    n = ct_1.shape[1]
    z = xt @ W
    f = torch.sigmoid(z[:, n:2 * n] + b[:n])
    r = torch.sigmoid(z[:, 2 * n:] + b[n:])
    c = f * ct_1 + (1 - f) * z[:, :n]
    return r * torch.tanh(c) + (1 - r) * xt, c


@op("sru", n_out=2)
def sru(x, W, b, c0, mask=None, **kw):
    """x [B, n, T], W [3n, n], b [2n], c0 [B, n] -> (h [B, n, T], c [B, n, T])."""
    B, n, T = x.shape
    xm = x * mask.unsqueeze(2) if mask is not None else x
    z = torch.einsum("kn,bnt->bkt", W, xm)
    c, hs, cs = c0, [], []
    for t in range(T):
        f = torch.sigmoid(z[:, n:2 * n, t] + b[:n])
        r = torch.sigmoid(z[:, 2 * n:, t] + b[n:])
        c = f * c + (1 - f) * z[:, :n, t]
        hs.append(r * torch.tanh(c) + (1 - r) * xm[:, :, t])
        cs.append(c)
    return torch.stack(hs, 2), torch.stack(cs, 2)


op("sru_bp", n_out=-1)(_autobp(lambda *a, **kw: sru(*a, **kw)[0], 4))


@op("sru_bi", n_out=2)
def sru_bi(x, W, b, c0, mask=None, **kw):
    """Bidirectional SRU: x [T, B, 2n], W [2n, 6n], b [4n], c0 [B, 2n] (``helpers/cuda/sru.cu`` sruBICuda)."""
    T, B, n2 = x.shape
    n = n2 // 2
    xm = x * mask.unsqueeze(0).unsqueeze(2) if mask is not None and mask.dim() == 1 else x
    z = (xm.reshape(T * B, n2) @ W).reshape(T, B, 2, 3, n)
    hs = torch.zeros_like(x)
    cs = torch.zeros_like(x)
    for d in range(2):
        c = c0[:, d * n:(d + 1) * n]
        bf, br = b[d * n:(d + 1) * n], b[2 * n + d * n:2 * n + (d + 1) * n]
        for t in (range(T) if d == 0 else range(T - 1, -1, -1)):
            zz = z[t, :, d]
            f = torch.sigmoid(zz[:, 1] + bf)
            r = torch.sigmoid(zz[:, 2] + br)
            c = f * c + (1 - f) * zz[:, 0]
            hs[t, :, d * n:(d + 1) * n] = r * torch.tanh(c) + (1 - r) * xm[t, :, d * n:(d + 1) * n]
            cs[t, :, d * n:(d + 1) * n] = c
    return hs, cs


op("sru_bi_bp", n_out=-1)(_autobp(lambda *a, **kw: sru_bi(*a, **kw)[0], 4))


def _simple_rnn(x, Wx, Wh, b, h0, seqLen=None, reverse=False):
    T, B, _ = x.shape
    n = Wh.shape[0]
    h = h0 if h0 is not None else torch.zeros(B, n, dtype=x.dtype, device=x.device)
    hs = [None] * T
    if b is not None and b.numel() == 2 * n:           # [2 * units]: input-to-hidden and hidden-to-hidden biases (helpers/impl/rnn.cpp:41)
        b = b.reshape(-1)[:n] + b.reshape(-1)[n:]
    for t in (range(T - 1, -1, -1) if reverse else range(T)):
        hn = torch.tanh(x[t] @ Wx + h @ Wh + b)
        if seqLen is not None:
            m = (t < seqLen).to(x.dtype).unsqueeze(1)
            hn = m * hn + (1 - m) * h
        hs[t] = hn
        h = hn
    return torch.stack(hs, 0), h


@op("static_rnn", n_out=2)
def static_rnn(x, Wx, Wh, b, h0=None, maxTimeStep=None, **kw):
    return _simple_rnn(x, Wx, Wh, b, h0, maxTimeStep)


@op("dynamic_rnn", n_out=2)
def dynamic_rnn(x, Wx, Wh, b, h0=None, maxTimeStep=None, timeMajor=False, **kw):
    xt = x if timeMajor else x.permute(1, 0, 2)
    hs, h = _simple_rnn(xt, Wx, Wh, b, h0, maxTimeStep)
    return (hs if timeMajor else hs.permute(1, 0, 2)), h


@op("static_bidirectional_rnn", n_out=3)
def static_bidirectional_rnn(x, WxFW, WhFW, bFW, WxBW, WhBW, bBW, h0FW=None, h0BW=None, maxTimeStep=None, **kw):
    f, hf = _simple_rnn(x, WxFW, WhFW, bFW, h0FW, maxTimeStep)
    r, hb = _simple_rnn(x, WxBW, WhBW, bBW, h0BW, maxTimeStep, reverse=True)
    return torch.cat([f, r], -1), hf, hb


@op("dynamic_bidirectional_rnn", n_out=4)
def dynamic_bidirectional_rnn(x, WxFW, WhFW, bFW, WxBW, WhBW, bBW, h0FW=None, h0BW=None, maxTimeStep=None, timeMajor=False, **kw):
    xt = x if timeMajor else x.permute(1, 0, 2)
    f, hf = _simple_rnn(xt, WxFW, WhFW, bFW, h0FW, maxTimeStep)
    r, hb = _simple_rnn(xt, WxBW, WhBW, bBW, h0BW, maxTimeStep, reverse=True)
    if not timeMajor:
        f, r = f.permute(1, 0, 2), r.permute(1, 0, 2)
    return f, r, hf, hb
