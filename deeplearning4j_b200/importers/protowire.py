"""Minimal protobuf wire-format reader / writer used by the ONNX and TensorFlow importers (neither ``onnx`` nor
``tensorflow`` is needed): messages are decoded into ``{field number: [values]}`` with nested messages decoded
lazily by the caller, and encoded from (field, wire type, value) triples."""
from __future__ import annotations

import struct


def read_varint(buf, pos):
    result, shift = 0, 0
    while True:
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not b & 0x80:
            return result, pos
        shift += 7


def decode(buf) -> dict:
    """{field: [value, ...]}; varints as int, 64/32-bit as raw bytes, length-delimited as bytes / memoryview."""
    mv = memoryview(buf)
    out, pos, n = {}, 0, len(mv)
    while pos < n:
        key, pos = read_varint(mv, pos)
        field, wt = key >> 3, key & 7
        if wt == 0:
            v, pos = read_varint(mv, pos)
        elif wt == 1:
            v, pos = bytes(mv[pos:pos + 8]), pos + 8
        elif wt == 2:
            ln, pos = read_varint(mv, pos)
            v, pos = mv[pos:pos + ln], pos + ln
        elif wt == 5:
            v, pos = bytes(mv[pos:pos + 4]), pos + 4
        else:
            raise ValueError(f"unsupported protobuf wire type {wt}")
        out.setdefault(field, []).append(v)
    return out


def signed(v, bits=64):
    return v - (1 << bits) if v >= (1 << (bits - 1)) else v


def packed_varints(vals):
    """Values of a repeated varint field: both packed (bytes) and unpacked (ints) encodings are accepted."""
    out = []
    for v in vals:
        if isinstance(v, int):
            out.append(signed(v))
        else:
            pos, mv = 0, memoryview(v)
            while pos < len(mv):
                x, pos = read_varint(mv, pos)
                out.append(signed(x))
    return out


def packed_fixed(vals, fmt):
    out = []
    for v in vals:                       # one fixed-width value (unpacked encoding) or a packed run of them
        out.extend(x[0] for x in struct.iter_unpack("<" + fmt, bytes(v)))
    return out


def string(v):
    return bytes(v).decode("utf-8")


# ----------------------------------------------------------------------------- writer
def _varint(v):
    if v < 0:
        v += 1 << 64
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        out.append(b | (0x80 if v else 0))
        if not v:
            return bytes(out)


def field_varint(f, v): return _varint(f << 3) + _varint(int(v))
def field_bytes(f, b): return _varint((f << 3) | 2) + _varint(len(b)) + bytes(b)
def field_string(f, s): return field_bytes(f, s.encode("utf-8"))
def field_float(f, v): return _varint((f << 3) | 5) + struct.pack("<f", v)
def field_packed_varints(f, vals): return field_bytes(f, b"".join(_varint(int(v)) for v in vals))
def field_packed_floats(f, vals): return field_bytes(f, struct.pack(f"<{len(vals)}f", *vals))
