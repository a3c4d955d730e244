"""Threshold ("flexible") and bitmap gradient codecs — host reference and device dispatch.

Semantics follow the surviving native codec of the reference
(``libnd4j/include/loops/impl/type_conversions.cpp:92-190`` CPU,
``libnd4j/include/loops/cuda/type_conversions.cu:215-500`` CUDA) and the Java constants in
``nd4j-api/.../linalg/compression/ThresholdCompression.java:22-25``:

* message = ``int32[4 + payload]`` with header ``[k, N, float_bits(tau), flag]``,
  ``flag`` 0 = FLEXIBLE (sparse), 1 = BITMAP;
* sparse payload: ``+(i+1)`` / ``-(i+1)`` for every ``|x[i]| >= tau`` in ascending index order;
  the source keeps the residual ``x[i] -/+ tau``; encoding stops after ``capacity`` entries;
* bitmap payload: one word per 16 elements, bit ``b`` = ``|x| >= tau``, bit ``b+16`` = negative;
  a negative value with ``tau/2 <= |x| < tau`` sets only the sign bit and moves by ``+tau/2``;
* decode accumulates (``target[i] += +/-tau``), so several messages can be summed into one buffer.

The torch implementations below run on CPU tensors (gloo ranks, tests) and are the oracle for
the CUDA kernels; CUDA tensors go to ``ops.native``.
"""
from __future__ import annotations

import struct

import torch

FLEXIBLE_ENCODING = 0
BITMAP_ENCODING = 1


def _bits(tau: float) -> int:
    return struct.unpack("<i", struct.pack("<f", float(tau)))[0]


def _tau_of(msg) -> float:
    return struct.unpack("<f", struct.pack("<i", int(msg[2])))[0]


def threshold_encode(x: torch.Tensor, tau: float, capacity: int | None = None) -> torch.Tensor:
    """Encode fp32 ``x`` in place (residual stays in ``x``) and return the int32 message."""
    flat = x.view(-1)
    n = flat.numel()
    if flat.is_cuda:
        from ..ops import native
        return native.threshold_encode(flat, tau, capacity)
    cap = n if capacity is None else int(capacity)
    idx = torch.nonzero(flat.abs() >= tau, as_tuple=False).view(-1)
    total = idx.numel()
    idx = idx[:cap]
    vals = flat[idx]
    neg = vals < 0
    payload = (idx + 1).to(torch.int32)
    payload = torch.where(neg, -payload, payload)
    flat[idx] = vals + torch.where(neg, torch.full_like(vals, tau), torch.full_like(vals, -tau))
    head = torch.tensor([min(total, cap), n, _bits(tau), FLEXIBLE_ENCODING], dtype=torch.int32)
    return torch.cat([head, payload])


def threshold_decode(msg: torch.Tensor, target: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    flat = target.view(-1)
    if flat.is_cuda:
        from ..ops import native
        return native.threshold_decode(msg, flat, scale, atomics=False)
    k = min(int(msg[0]), msg.numel() - 4)
    if k <= 0:
        return target
    tau = _tau_of(msg) * scale
    e = msg[4:4 + k].to(torch.int64)
    idx = e.abs() - 1
    flat.index_add_(0, idx, torch.where(e < 0, -tau, tau).to(flat.dtype))
    return target


def bitmap_encode(x: torch.Tensor, tau: float) -> torch.Tensor:
    flat = x.view(-1)
    n = flat.numel()
    if flat.is_cuda:
        from ..ops import native
        return native.bitmap_encode(flat, tau)
    a = flat.abs()
    big = a >= tau
    neg = flat < 0
    half = (~big) & neg & (a >= tau / 2)
    val_bits = big.to(torch.int64)
    sign_bits = ((big & neg) | half).to(torch.int64)
    flat.add_(torch.where(big, torch.where(neg, tau, -tau), torch.where(half, tau / 2, 0.0)).to(flat.dtype))
    words = (n + 15) // 16
    pad = words * 16 - n
    if pad:
        val_bits = torch.nn.functional.pad(val_bits, [0, pad])
        sign_bits = torch.nn.functional.pad(sign_bits, [0, pad])
    sh = torch.arange(16, dtype=torch.int64)
    w = ((val_bits.view(words, 16) << sh).sum(1) | ((sign_bits.view(words, 16) << (sh + 16)).sum(1)))
    w = torch.where(w >= 2 ** 31, w - 2 ** 32, w).to(torch.int32)
    head = torch.tensor([int(big.sum() + half.sum()), n, _bits(tau), BITMAP_ENCODING], dtype=torch.int32)
    return torch.cat([head, w])


def bitmap_decode(msg: torch.Tensor, target: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    flat = target.view(-1)
    n = flat.numel()
    if flat.is_cuda:
        from ..ops import native
        return native.bitmap_decode(msg, flat, scale)
    tau = _tau_of(msg) * scale
    words = (n + 15) // 16
    w = msg[4:4 + words].to(torch.int64) & 0xFFFFFFFF
    sh = torch.arange(16, dtype=torch.int64)
    bit = ((w.unsqueeze(1) >> sh) & 1).bool().view(-1)[:n]
    sign = ((w.unsqueeze(1) >> (sh + 16)) & 1).bool().view(-1)[:n]
    delta = torch.where(bit, torch.where(sign, -tau, tau), torch.where(sign, -tau / 2, 0.0))
    flat.add_(delta.to(flat.dtype))
    return target


def encode(x: torch.Tensor, tau: float, capacity: int | None = None, force: int | None = None) -> torch.Tensor:
    """Pick the smaller representation the way ``EncodingHandler`` did: sparse costs ``4*(k+4)``
    bytes, bitmap ``4*(N/16+4)`` bytes, so bitmap wins when more than 1/16 of the entries fire."""
    flat = x.view(-1)
    if force == BITMAP_ENCODING:
        return bitmap_encode(flat, tau)
    if force == FLEXIBLE_ENCODING:
        return threshold_encode(flat, tau, capacity)
    k = int((flat.abs() >= tau).sum())
    if k > flat.numel() // 16:
        return bitmap_encode(flat, tau)
    return threshold_encode(flat, tau, capacity)


def decode(msg: torch.Tensor, target: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    if int(msg[3]) == BITMAP_ENCODING:
        return bitmap_decode(msg, target, scale)
    return threshold_decode(msg, target, scale)
