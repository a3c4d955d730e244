"""SDNB container and SDZ archive for SameDiff graphs.

Parity: ``autodiff/samediff/serde/SameDiffSerializer.java`` (container layout ``:78-100,649-950``,
sharding ``:224-430,531-552``) and ``SDZSerializer.java`` (ZIP of the ``.sdnb`` files).

File layout (all header integers big-endian):
``"SDNB" | int32 version=1 | int64 manifestOffset | int64 manifestLength | int64 metadataOffset=32 |
FlatGraph bytes | raw array blobs | manifest``.  Arrays of 1 MiB or more are left out of the FlatGraph
(their FlatArray keeps shape and dtype, no buffer) and appended raw; the manifest maps variable name ->
(file offset, byte length) and is a Java-serialised ``LinkedHashMap<String, Pair<Long, Long>>`` so that
JVM readers can consume it.  Models larger than the shard limit are split: shard 0 holds the graph,
further shards hold variables only, named ``<base>.shard<k>-of-<n>.sdnb``.
"""
from __future__ import annotations

import io
import os
import struct
import tempfile
import zipfile

import numpy as np
import torch

from . import flatbuffers as fb
from . import flatgraph

MAGIC = b"SDNB"
VERSION = 1
HEADER_SIZE = 32
APPEND_THRESHOLD_BYTES = 1 << 20
MAX_SHARD_FILE_BYTES = 1 << 30


# ----------------------------------------------------------------------------- java.io.Serializable subset
_TC_NULL, _TC_REFERENCE, _TC_CLASSDESC, _TC_OBJECT, _TC_STRING, _TC_BLOCKDATA, _TC_ENDBLOCKDATA = 0x70, 0x71, 0x72, 0x73, 0x74, 0x77, 0x78
_BASE_HANDLE = 0x7E0000
_UID = {"java.util.LinkedHashMap": 3801124242820219131, "java.util.HashMap": 362498820763181265,
        "org.nd4j.common.primitives.Pair": 119, "java.lang.Long": 4290774380558885855, "java.lang.Number": -8742448824652078965}


class _JavaOut:
    """Writes exactly the object graph LinkedHashMap<String, Pair<Long, Long>> in Java serialization protocol 2."""

    def __init__(self):
        self.b = io.BytesIO()
        self.handles = {}
        self.next = _BASE_HANDLE
        self.b.write(struct.pack(">HH", 0xACED, 5))

    def _new_handle(self, key=None):
        h = self.next
        self.next += 1
        if key is not None:
            self.handles[key] = h
        return h

    def _utf(self, s):
        raw = s.encode("utf-8")
        self.b.write(struct.pack(">H", len(raw)) + raw)

    def _class_desc(self, name, flags, fields, parent=None):
        if ("class", name) in self.handles:
            self.b.write(struct.pack(">BI", _TC_REFERENCE, self.handles[("class", name)]))
            return
        self.b.write(bytes([_TC_CLASSDESC]))
        self._utf(name)
        self.b.write(struct.pack(">q", _UID[name]))
        self._new_handle(("class", name))
        self.b.write(struct.pack(">BH", flags, len(fields)))
        for tcode, fname, sig in fields:
            self.b.write(tcode.encode())
            self._utf(fname)
            if sig is not None:
                self._string(sig)
        self.b.write(bytes([_TC_ENDBLOCKDATA]))
        if parent is None:
            self.b.write(bytes([_TC_NULL]))
        else:
            parent()

    def _string(self, s):
        if ("str", s) in self.handles:
            self.b.write(struct.pack(">BI", _TC_REFERENCE, self.handles[("str", s)]))
            return
        self.b.write(bytes([_TC_STRING]))
        self._utf(s)
        self._new_handle(("str", s))

    def _long(self, v):
        self.b.write(bytes([_TC_OBJECT]))
        self._class_desc("java.lang.Long", 0x02, [("J", "value", None)],
                         parent=lambda: self._class_desc("java.lang.Number", 0x02, []))
        self._new_handle()
        self.b.write(struct.pack(">q", v))

    def _pair(self, a, b):
        self.b.write(bytes([_TC_OBJECT]))
        self._class_desc("org.nd4j.common.primitives.Pair", 0x02,
                         [("L", "key", "Ljava/lang/Object;"), ("L", "value", "Ljava/lang/Object;")])
        self._new_handle()
        self._long(a)
        self._long(b)

    def linked_hash_map(self, m):
        self.b.write(bytes([_TC_OBJECT]))
        self._class_desc("java.util.LinkedHashMap", 0x02, [("Z", "accessOrder", None)],
                         parent=lambda: self._class_desc("java.util.HashMap", 0x03, [("F", "loadFactor", None), ("I", "threshold", None)]))
        self._new_handle()
        cap = 16
        while cap * 0.75 < len(m):
            cap *= 2
        self.b.write(struct.pack(">fi", 0.75, int(cap * 0.75)))          # HashMap default fields
        self.b.write(struct.pack(">BBii", _TC_BLOCKDATA, 8, cap, len(m)))  # HashMap.writeObject: buckets, size
        for k, (off, ln) in m.items():
            self._string(k)
            self._pair(int(off), int(ln))
        self.b.write(bytes([_TC_ENDBLOCKDATA]))
        self.b.write(struct.pack(">?", False))                             # LinkedHashMap.accessOrder
        return self.b.getvalue()


class _JavaIn:
    def __init__(self, data):
        self.d, self.p = bytes(data), 0
        self.handles = []
        magic, ver = struct.unpack_from(">HH", self.d, 0)
        if magic != 0xACED:
            raise ValueError("manifest is not a Java serialization stream")
        self.p = 4

    def _take(self, fmt):
        v = struct.unpack_from(fmt, self.d, self.p)
        self.p += struct.calcsize(fmt)
        return v if len(v) > 1 else v[0]

    def _utf(self):
        n = self._take(">H")
        s = self.d[self.p:self.p + n].decode("utf-8")
        self.p += n
        return s

    def _class_desc(self):
        tc = self._take(">B")
        if tc == _TC_NULL:
            return None
        if tc == _TC_REFERENCE:
            return self.handles[self._take(">I") - _BASE_HANDLE]
        assert tc == _TC_CLASSDESC, hex(tc)
        name = self._utf()
        self._take(">q")
        desc = {"name": name, "fields": []}
        self.handles.append(desc)
        desc["flags"], nf = self._take(">BH")
        for _ in range(nf):
            t = chr(self._take(">B"))
            fname = self._utf()
            if t in "L[":
                self._object()
            desc["fields"].append((t, fname))
        assert self._take(">B") == _TC_ENDBLOCKDATA
        desc["parent"] = self._class_desc()
        return desc

    def _object(self):
        tc = self._take(">B")
        if tc == _TC_NULL:
            return None
        if tc == _TC_REFERENCE:
            return self.handles[self._take(">I") - _BASE_HANDLE]
        if tc == _TC_STRING:
            s = self._utf()
            self.handles.append(s)
            return s
        assert tc == _TC_OBJECT, hex(tc)
        desc = self._class_desc()
        slot = len(self.handles)
        self.handles.append(None)
        chain = []
        d = desc
        while d is not None:
            chain.append(d)
            d = d["parent"]
        vals = {}
        obj = None
        for d in reversed(chain):
            for t, fname in d["fields"]:
                vals[fname] = self._object() if t in "L[" else self._take({"J": ">q", "I": ">i", "F": ">f", "Z": ">?", "D": ">d", "B": ">b", "S": ">h", "C": ">H"}[t])
            if d["name"] == "java.util.HashMap":
                tcb, ln = self._take(">BB")
                assert tcb == _TC_BLOCKDATA and ln == 8
                _, size = self._take(">ii")
                obj = {}
                for _ in range(size):
                    k = self._object()
                    obj[k] = self._object()
                assert self._take(">B") == _TC_ENDBLOCKDATA
        name = desc["name"]
        if name == "java.lang.Long":
            obj = vals["value"]
        elif name == "org.nd4j.common.primitives.Pair":
            obj = (vals["key"], vals["value"])
        self.handles[slot] = obj
        return obj

    def read(self):
        return self._object()


def write_manifest(m: dict) -> bytes:
    return _JavaOut().linked_hash_map(m)


def read_manifest(data) -> dict:
    return _JavaIn(data).read() or {}


# ----------------------------------------------------------------------------- container
def _write_container(path, graph_bytes: bytes, blobs: dict):
    """blobs: name -> contiguous CPU tensor appended raw after the FlatGraph."""
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack(">iqqq", VERSION, -1, -1, HEADER_SIZE))
        f.write(graph_bytes)
        manifest = {}
        for name, t in blobs.items():
            raw = flatgraph.flat_array(t)["buffer"]
            manifest[name] = (f.tell(), len(raw))
            f.write(raw)
        moff = f.tell()
        mb = write_manifest(manifest)
        f.write(mb)
        f.seek(8)
        f.write(struct.pack(">qq", moff, len(mb)))


def _read_container(path):
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(HEADER_SIZE)
        if len(head) < HEADER_SIZE or head[:4] != MAGIC:
            raise IOError(f"{path}: not an SDNB file")
        ver, moff, mlen, goff = struct.unpack(">iqqq", head[4:])
        if ver != VERSION:
            raise IOError(f"{path}: unsupported SDNB version {ver}")
        if goff != HEADER_SIZE or moff < goff or mlen < 0 or moff + mlen > size:
            raise IOError(f"{path}: corrupt SDNB header")
        f.seek(moff)
        manifest = read_manifest(f.read(mlen)) if mlen else {}
        first_blob = min([o for o, _ in manifest.values()] + [moff])
        f.seek(goff)
        graph_bytes = f.read(first_blob - goff)
    return graph_bytes, manifest


def _read_blob(path, off, ln, dtype_fb, shape):
    with open(path, "rb") as f:
        f.seek(off)
        raw = f.read(ln)
    return flatgraph.from_flat_array({"dtype": dtype_fb, "shape": shape, "buffer": raw, "byteOrder": 0})


def _split(sd, threshold):
    """Graph dict pieces: the SameDiff with large arrays detached, and the detached arrays."""
    from ..core import VariableType
    large = {}
    for n, v in sd.variables.items():
        if v.variableType in (VariableType.VARIABLE, VariableType.CONSTANT):
            a = sd.arrays.get(n)
            if a is not None and a.numel() * a.element_size() >= threshold:
                large[n] = a
    return large


def save(sd, path, saveUpdaterState=True, maxShardBytes=MAX_SHARD_FILE_BYTES, appendThreshold=APPEND_THRESHOLD_BYTES):
    large = _split(sd, appendThreshold)
    g = fb.decode("FlatGraph", flatgraph.to_flatbuffers(_without(sd, large), saveUpdaterState))
    # restore shape / dtype of the detached arrays so readers know what the blobs hold
    for fv in g["variables"]:
        if fv["name"] in large:
            a = large[fv["name"]]
            fv["ndarray"] = {"shape": list(a.shape), "dtype": flatgraph._DT_TO_FB[flatgraph.DataType.from_torch(a.dtype)], "byteOrder": 0}
    meta = {"nd4j.format.version": str(VERSION), "nd4j.format.type": "APPENDED_BLOB", "framework.version": "deeplearning4j_b200"}
    keys = list(g["metadataKeys"] or []) + [k for k in meta if k not in (g["metadataKeys"] or [])]
    vals = list(g["metadataValues"] or []) + [meta[k] for k in keys[len(g["metadataValues"] or []):]]
    g["metadataKeys"], g["metadataValues"] = keys, vals
    graph_bytes = fb.encode("FlatGraph", g)
    total = len(graph_bytes) + sum(a.numel() * a.element_size() for a in large.values())
    if total + HEADER_SIZE <= maxShardBytes:
        _write_container(path, graph_bytes, large)
        return [path]
    # sharded: graph in shard 0, variables spread over the following shards
    shards, cur, cur_bytes = [], {}, 0
    for n, a in large.items():
        nb = a.numel() * a.element_size()
        if cur and cur_bytes + nb > maxShardBytes:
            shards.append(cur)
            cur, cur_bytes = {}, 0
        cur[n] = a
        cur_bytes += nb
    if cur:
        shards.append(cur)
    total_shards = len(shards) + 1
    base = path[:-5] if path.endswith(".sdnb") else path
    files = [f"{base}.shard0-of-{total_shards}.sdnb"]
    _write_container(files[0], graph_bytes, {})
    for k, blobs in enumerate(shards, start=1):
        sg = {"id": 119, "variables": [fv for fv in g["variables"] if fv["name"] in blobs],
              "metadataKeys": ["shard.index", "shard.type"], "metadataValues": [str(k), "VARIABLES"]}
        fn = f"{base}.shard{k}-of-{total_shards}.sdnb"
        _write_container(fn, fb.encode("FlatGraph", sg), blobs)
        files.append(fn)
    return files


def _without(sd, large):
    """A shallow copy of ``sd`` whose large arrays are hidden from the FlatGraph writer."""
    if not large:
        return sd
    import copy
    c = copy.copy(sd)
    c.arrays = {k: v for k, v in sd.arrays.items() if k not in large}
    return c


def _attach_blobs(sd, path, graph_dict, manifest):
    info = {fv["name"]: fv["ndarray"] for fv in graph_dict["variables"] or [] if fv["ndarray"] is not None}
    for name, (off, ln) in manifest.items():
        fa = info.get(name)
        if fa is None:
            continue
        sd.arrays[name] = _read_blob(path, off, ln, fa["dtype"], fa["shape"])


def load(path, loadUpdaterState=True):
    files = [path]
    if not os.path.exists(path):
        base = path[:-5] if path.endswith(".sdnb") else path
        d = os.path.dirname(base) or "."
        pref = os.path.basename(base) + ".shard"
        found = sorted(f for f in os.listdir(d) if f.startswith(pref) and f.endswith(".sdnb"))
        if not found:
            raise FileNotFoundError(path)
        n = int(found[0].rsplit("-of-", 1)[1][:-5])
        files = [os.path.join(d, f"{os.path.basename(base)}.shard{k}-of-{n}.sdnb") for k in range(n)]
        for f in files:
            if not os.path.exists(f):
                raise FileNotFoundError(f"missing shard {f}")
    graph_bytes, manifest = _read_container(files[0])
    g = fb.decode("FlatGraph", graph_bytes)
    large_names = {fv["name"] for fv in g["variables"] or []
                   if fv["ndarray"] is not None and (fv["ndarray"]["buffer"] is None or len(fv["ndarray"]["buffer"]) == 0)
                   and int(np.prod(fv["ndarray"]["shape"] if fv["ndarray"]["shape"] is not None else [1])) > 0}
    sd = flatgraph.from_flatbuffers(graph_bytes, loadUpdaterState=False)
    for n in large_names:
        sd.arrays.pop(n, None)
    _attach_blobs(sd, files[0], g, manifest)
    for f in files[1:]:
        gb, mf = _read_container(f)
        _attach_blobs(sd, f, fb.decode("FlatGraph", gb), mf)
    missing = [n for n in large_names if n not in sd.arrays]
    if missing:
        raise IOError(f"arrays missing from the container: {missing[:5]}")
    if loadUpdaterState and g["updaterState"]:
        _load_updater_state(sd, g)
    return sd


def _load_updater_state(sd, g):
    from ..training import _ensure_state
    if sd.trainingConfig is None:
        return
    st = _ensure_state(sd)
    state = st.updater.state
    by_param = {u["paramName"]: u for u in g["updaterState"]}
    for b in st.updater.blocks:
        n = b.numel
        for e in b.entries:
            u = by_param.get(e.spec.name)
            if u is None:
                continue
            rel = e.offset - b.start
            for k, fa in enumerate(u["updaterStateValues"] or []):
                dst = state[b.state_offset + k * n + rel: b.state_offset + k * n + rel + e.spec.numel]
                dst.copy_(flatgraph.from_flat_array(fa).reshape(-1).to(dst.dtype))


# ----------------------------------------------------------------------------- SDZ
def save_sdz(sd, path, saveUpdaterState=True, **kw):
    with tempfile.TemporaryDirectory() as tmp:
        files = save(sd, os.path.join(tmp, "model.sdnb"), saveUpdaterState, **kw)
        with zipfile.ZipFile(path, "w", zipfile.ZIP_DEFLATED) as z:
            for f in files:
                z.write(f, os.path.basename(f))


def load_sdz(path, loadUpdaterState=True):
    with tempfile.TemporaryDirectory() as tmp:
        with zipfile.ZipFile(path) as z:
            for info in z.infolist():
                name = os.path.basename(info.filename)
                if not name or not name.endswith(".sdnb"):
                    continue
                with z.open(info) as src, open(os.path.join(tmp, name), "wb") as dst:
                    head = src.read(4)
                    if head != MAGIC:
                        continue
                    dst.write(head)
                    while True:
                        chunk = src.read(1 << 22)
                        if not chunk:
                            break
                        dst.write(chunk)
        return load(os.path.join(tmp, "model.sdnb"), loadUpdaterState)
