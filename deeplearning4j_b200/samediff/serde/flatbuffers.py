"""A small schema-driven FlatBuffers encoder / decoder (little-endian wire format, vtables, forward
unsigned offsets) plus the ND4J graph schema (``libnd4j/include/graph/scheme/{array,utils,variable,
node,properties,config,graph}.fbs``) expressed as Python tables.

The encoder lays objects out front to back: a table is written first (its vtable directly before it),
then every object it refers to, and the 32-bit forward offsets are patched in afterwards.  That order
is valid FlatBuffers (readers only require referents to sit at higher addresses than the referring
field) and keeps the writer allocation-light for the half-gigabyte parameter arrays of a large graph.
"""
from __future__ import annotations

import struct

import numpy as np

_SCALARS = {"byte": ("<b", 1), "ubyte": ("<B", 1), "bool": ("<?", 1), "short": ("<h", 2), "ushort": ("<H", 2),
            "int": ("<i", 4), "uint": ("<I", 4), "float": ("<f", 4), "long": ("<q", 8), "ulong": ("<Q", 8), "double": ("<d", 8)}
_NP = {"byte": np.int8, "ubyte": np.uint8, "bool": np.bool_, "short": "<i2", "ushort": "<u2", "int": "<i4", "uint": "<u4",
       "float": "<f4", "long": "<i8", "ulong": "<u8", "double": "<f8"}


def vec(t):
    return ("vec", t)


def table(name):
    return ("table", name)


# field order == field id (schema declaration order)
SCHEMA = {
    "BufferChunk": [("index", "long"), ("data", vec("byte"))],
    "FlatArray": [("shape", vec("long")), ("buffer", vec("byte")), ("dtype", "byte"), ("byteOrder", "byte"),
                  ("bufferChunks", vec(table("BufferChunk"))), ("totalBufferSize", "long"),
                  ("externalDataFilename", vec("string")), ("isExternal", "bool")],
    "LongPair": [("first", "long"), ("second", "long")],
    "LongTriple": [("first", "long"), ("second", "long"), ("third", "long")],
    "IntPair": [("first", "int"), ("second", "int")],
    "IntTriple": [("first", "int"), ("second", "int"), ("third", "int")],
    "FlatVariable": [("id", table("IntPair")), ("name", "string"), ("dtype", "byte"), ("shape", vec("long")),
                     ("ndarray", table("FlatArray")), ("device", "int"), ("variabletype", "byte"),
                     ("controlDeps", vec("string")), ("controlDepForOp", vec("string")), ("controlDepsForVar", vec("string"))],
    "FlatProperties": [("name", "string"), ("i", vec("int")), ("l", vec("long")), ("d", vec("double")),
                       ("a", vec(table("FlatArray"))), ("b", vec("bool")), ("s", vec("string")), ("shape", vec("int"))],
    "FlatNode": [("id", "int"), ("name", "string"), ("opType", "byte"), ("opNum", "long"),
                 ("properties", vec(table("FlatProperties"))), ("input", vec("int")), ("inputPaired", vec(table("IntPair"))),
                 ("output", vec("int")), ("extraParams", vec("double")), ("extraInteger", vec("long")), ("extraBools", vec("bool")),
                 ("dimensions", vec("int")), ("device", "int"), ("scope_id", "int"), ("scope_name", "string"),
                 ("outputNames", vec("string")), ("opName", "string"), ("outputTypes", vec("byte")), ("scalar", table("FlatArray")),
                 ("controlDeps", vec("string")), ("varControlDeps", vec("string")), ("controlDepFor", vec("string")),
                 ("extraTypes", vec("byte")), ("extraStrings", vec("string"))],
    "FlatConfiguration": [("id", "long"), ("executionMode", "byte"), ("profilingMode", "byte"), ("outputMode", "byte"),
                          ("timestats", "bool"), ("footprintForward", "long"), ("footprintBackward", "long"), ("direction", "byte")],
    "UpdaterState": [("paramName", "string"), ("updaterStateKeys", vec("string")), ("updaterStateValues", vec(table("FlatArray")))],
    "SameDiffSubInstance": [("name", "string"), ("serializedData", vec("ubyte"))],
    "FlatGraph": [("id", "long"), ("variables", vec(table("FlatVariable"))), ("nodes", vec(table("FlatNode"))),
                  ("outputs", vec(table("IntPair"))), ("configuration", table("FlatConfiguration")), ("placeholders", vec("string")),
                  ("lossVariables", vec("string")), ("trainingConfig", "string"), ("updaterState", vec(table("UpdaterState"))),
                  ("metadataKeys", vec("string")), ("metadataValues", vec("string")), ("subInstances", vec(table("SameDiffSubInstance")))],
}

# enum values (array.fbs, utils.fbs, variable.fbs)
DTYPE = {"INHERIT": 0, "BOOL": 1, "FLOAT8": 2, "HALF": 3, "HALF2": 4, "FLOAT": 5, "DOUBLE": 6, "INT8": 7, "INT16": 8, "INT32": 9,
         "INT64": 10, "UINT8": 11, "UINT16": 12, "UINT32": 13, "UINT64": 14, "QINT8": 15, "QINT16": 16, "BFLOAT16": 17,
         "UTF8": 50, "UTF16": 51, "UTF32": 52}
OPTYPE = {"TRANSFORM_FLOAT": 0, "TRANSFORM_SAME": 1, "TRANSFORM_BOOL": 2, "TRANSFORM_STRICT": 3, "TRANSFORM_ANY": 4, "REDUCE_FLOAT": 5,
          "REDUCE_SAME": 6, "REDUCE_LONG": 7, "REDUCE_BOOL": 8, "INDEX_REDUCE": 9, "SCALAR": 10, "SCALAR_BOOL": 11, "BROADCAST": 12,
          "BROADCAST_BOOL": 13, "PAIRWISE": 14, "PAIRWISE_BOOL": 15, "REDUCE_3": 16, "SUMMARYSTATS": 17, "SHAPE": 18, "AGGREGATION": 19,
          "RANDOM": 20, "CUSTOM": 21, "GRAPH": 22, "VARIABLE": 40, "BOOLEAN": 60, "LOGIC": 119, "UDF": 120}
VARTYPE = {"VARIABLE": 0, "CONSTANT": 1, "ARRAY": 2, "PLACEHOLDER": 3}


def _is_scalar(t):
    return isinstance(t, str) and t in _SCALARS


def union(type_field, members):
    """A union field: ``type_field`` names the ubyte field (declared just before it) holding the member id, ``members`` maps
    member ids to table names."""
    return ("union", type_field, members)


class _Writer:
    def __init__(self, schema=None):
        self.buf = bytearray()
        self.schema = SCHEMA if schema is None else schema

    def pad_to(self, align, bias=0):
        """Pad so that (len(buf) + bias) is a multiple of ``align``."""
        r = (len(self.buf) + bias) % align
        if r:
            self.buf.extend(b"\0" * (align - r))

    def patch_offset(self, at, target):
        struct.pack_into("<I", self.buf, at, target - at)

    # each write_* returns the absolute position that offsets must point at
    def write_string(self, s):
        raw = s.encode("utf-8") if isinstance(s, str) else bytes(s)
        self.pad_to(4)
        pos = len(self.buf)
        self.buf.extend(struct.pack("<I", len(raw)))
        self.buf.extend(raw)
        self.buf.append(0)
        return pos

    def write_vector(self, elem, values):
        if _is_scalar(elem):
            fmt, size = _SCALARS[elem]
            if isinstance(values, (bytes, bytearray, memoryview)) and size == 1:
                raw, n = values, len(values)
            else:
                arr = np.ascontiguousarray(np.asarray(values, dtype=_NP[elem]))
                raw, n = arr.tobytes() if arr.nbytes < (1 << 20) else memoryview(arr).cast("B"), arr.size
            self.pad_to(max(size, 4), bias=4 if size > 4 else 0)
            pos = len(self.buf)
            self.buf.extend(struct.pack("<I", n))
            self.buf.extend(raw)
            return pos
        # vector of offsets (strings or tables)
        values = list(values)
        self.pad_to(4)
        pos = len(self.buf)
        self.buf.extend(struct.pack("<I", len(values)))
        slots = len(self.buf)
        self.buf.extend(b"\0" * (4 * len(values)))
        for k, v in enumerate(values):
            target = self.write_string(v) if elem == "string" else self.write_table(elem[1], v)
            self.patch_offset(slots + 4 * k, target)
        return pos

    def write_table(self, name, obj):
        fields = self.schema[name]
        present = []          # (field id, type, value)
        for fid, f in enumerate(fields):
            fname, ftype = f[0], f[1]
            v = obj.get(fname)
            if v is None:
                continue
            if _is_scalar(ftype) and v == (f[2] if len(f) > 2 else 0):
                continue                                     # defaults are not stored
            if not _is_scalar(ftype) and ftype != "string" and ftype[0] == "union":
                ftype = table(ftype[2][obj[ftype[1]]])        # the member the type field selects
            present.append((fid, ftype, v))
        # inline layout: soffset, then fields largest first
        def fsize(t):
            return _SCALARS[t][1] if _is_scalar(t) else 4
        order = sorted(present, key=lambda p: -fsize(p[1]))
        off, slots = 4, {}
        for fid, ftype, _ in order:
            sz = fsize(ftype)
            off = (off + sz - 1) // sz * sz
            slots[fid] = off
            off += sz
        tsize = off
        nf = (max(slots) + 1) if slots else 0
        vtsize = 4 + 2 * nf
        align = max([4] + [fsize(t) for _, t, _ in present])
        self.pad_to(2)
        self.pad_to(align, bias=vtsize)
        vpos = len(self.buf)
        self.buf.extend(struct.pack("<HH", vtsize, tsize))
        for fid in range(nf):
            self.buf.extend(struct.pack("<H", slots.get(fid, 0)))
        tpos = len(self.buf)
        self.buf.extend(b"\0" * tsize)
        struct.pack_into("<i", self.buf, tpos, tpos - vpos)
        deferred = []
        for fid, ftype, v in present:
            at = tpos + slots[fid]
            if _is_scalar(ftype):
                struct.pack_into(_SCALARS[ftype][0], self.buf, at, v)
            else:
                deferred.append((at, ftype, v))
        for at, ftype, v in deferred:
            if ftype == "string":
                target = self.write_string(v)
            elif ftype[0] == "table":
                target = self.write_table(ftype[1], v)
            else:
                target = self.write_vector(ftype[1], v)
            self.patch_offset(at, target)
        return tpos


def encode(root_table: str, obj: dict, schema=None, identifier=None) -> bytes:
    """``schema`` defaults to the ND4J graph schema; ``identifier`` is the optional 4-byte file identifier after the root offset."""
    w = _Writer(schema)
    w.buf.extend(b"\0\0\0\0")
    if identifier is not None:
        assert len(identifier) == 4
        w.buf.extend(identifier)
    root = w.write_table(root_table, obj)
    w.patch_offset(0, root)
    return bytes(w.buf)


class _Reader:
    def __init__(self, data, schema=None):
        self.schema = SCHEMA if schema is None else schema
        self.mv = memoryview(data).cast("B") if not isinstance(data, memoryview) else data
        self.data = data

    def u32(self, at):
        return struct.unpack_from("<I", self.mv, at)[0]

    def indirect(self, at):
        return at + self.u32(at)

    def string(self, at):
        n = self.u32(at)
        return bytes(self.mv[at + 4:at + 4 + n]).decode("utf-8")

    def vector(self, elem, at, raw_bytes):
        n = self.u32(at)
        start = at + 4
        if _is_scalar(elem):
            size = _SCALARS[elem][1]
            if size == 1 and elem != "bool" and raw_bytes:
                return self.mv[start:start + n]
            arr = np.frombuffer(self.mv, dtype=_NP[elem], count=n, offset=start)
            return arr if raw_bytes else arr.tolist()
        out = []
        for k in range(n):
            p = self.indirect(start + 4 * k)
            out.append(self.string(p) if elem == "string" else self.table(elem[1], p, raw_bytes))
        return out

    def table(self, name, tpos, raw_bytes):
        fields = self.schema[name]
        vpos = tpos - struct.unpack_from("<i", self.mv, tpos)[0]
        vtsize = struct.unpack_from("<H", self.mv, vpos)[0]
        nf = (vtsize - 4) // 2
        out = {}
        for fid, f in enumerate(fields):
            fname, ftype = f[0], f[1]
            slot = struct.unpack_from("<H", self.mv, vpos + 4 + 2 * fid)[0] if fid < nf else 0
            if slot == 0:
                if _is_scalar(ftype):
                    out[fname] = f[2] if len(f) > 2 else (False if ftype == "bool" else 0)
                else:
                    out[fname] = None
                continue
            at = tpos + slot
            if _is_scalar(ftype):
                out[fname] = struct.unpack_from(_SCALARS[ftype][0], self.mv, at)[0]
            elif ftype == "string":
                out[fname] = self.string(self.indirect(at))
            elif ftype[0] == "table":
                out[fname] = self.table(ftype[1], self.indirect(at), raw_bytes)
            elif ftype[0] == "union":
                member = ftype[2].get(out.get(ftype[1], 0))
                out[fname] = self.table(member, self.indirect(at), raw_bytes) if member is not None else None
            else:
                out[fname] = self.vector(ftype[1], self.indirect(at), raw_bytes)
        return out


def decode(root_table: str, data, raw_bytes=True, schema=None) -> dict:
    """Decode ``data`` into nested dicts.  With ``raw_bytes`` byte vectors come back as zero-copy
    memoryviews and other scalar vectors as numpy arrays; otherwise everything is plain lists."""
    r = _Reader(data, schema)
    return r.table(root_table, r.indirect(0), raw_bytes)
