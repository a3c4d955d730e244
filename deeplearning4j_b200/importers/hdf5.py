"""A small HDF5 reader and writer in plain Python, enough for Keras ``.h5`` model files, and ``Hdf5Archive`` on top of it
(``deeplearning4j-modelimport/.../keras/Hdf5Archive.java``: ``readAttributeAsJson``, ``readAttributeAsString``, ``readDataSet``,
``getGroups``, ``getDataSets``, ``hasAttribute``; the reference binds the HDF5 C library through JavaCPP).

Supported subset of the file format (HDF5 File Format Specification, the structures that h5py / the HDF5 1.8+ library write by
default): superblock versions 0 and 1, version-1 object headers with continuation blocks, old-style groups (symbol-table message,
version-1 B-tree, ``SNOD`` nodes, local heap), dataspace messages v1 / v2, datatype classes fixed-point, floating-point, string and
variable-length string, contiguous, compact and chunked data layouts (B-tree-indexed chunks with the deflate, shuffle and fletcher32
filters), attribute messages v1 - v3, global heap collections for variable-length data.  New-style groups (link messages, fractal
heaps: ``libver='latest'``), other filters and superblock versions 2 / 3 raise ``Hdf5FormatError`` with the name of the unsupported structure.
"""
from __future__ import annotations

import struct

import numpy as np

SIGNATURE = b"\x89HDF\r\n\x1a\n"
UNDEF = 0xFFFFFFFFFFFFFFFF


class Hdf5FormatError(ValueError):
    pass


# ----------------------------------------------------------------------------- datatypes
def _decode_datatype(buf, at=0):
    """-> (kind, numpy dtype or None, size, extra).  kind: 'num', 'str' (fixed length), 'vlen_str'."""
    cls_ver = buf[at]
    cls, b0, b1, b2 = cls_ver & 0x0F, buf[at + 1], buf[at + 2], buf[at + 3]
    size = struct.unpack_from("<I", buf, at + 4)[0]
    if cls == 0:
        order = ">" if b0 & 1 else "<"
        return "num", np.dtype(f"{order}{'i' if b0 & 8 else 'u'}{size}"), size, None
    if cls == 1:
        order = ">" if b0 & 1 else "<"
        return "num", np.dtype(f"{order}f{size}"), size, None
    if cls == 3:
        return "str", np.dtype(f"S{size}"), size, {"pad": b0 & 0x0F, "utf8": (b0 >> 4) & 0x0F == 1}
    if cls == 9:
        if b0 & 0x0F != 1:
            raise Hdf5FormatError("variable-length sequences (only variable-length strings are supported)")
        return "vlen_str", None, size, None
    raise Hdf5FormatError(f"datatype class {cls}")


def _encode_datatype(dt):
    """Datatype message body for a numpy dtype ('S<n>' = fixed string), or the string 'vlen_str'."""
    if isinstance(dt, str) and dt == "vlen_str":
        base = struct.pack("<BBBBI", 0x13, 0x00, 0, 0, 1)                     # one-byte null-terminated ASCII string
        return struct.pack("<BBBBI", 0x19, 0x01, 0x01, 0, 16) + base          # class 9 v1: string, null-terminated, UTF-8
    dt = np.dtype(dt)
    if dt.kind == "S":
        return struct.pack("<BBBBI", 0x13, 0x01, 0, 0, dt.itemsize)           # null-padded ASCII
    if dt.kind in "iu":
        return struct.pack("<BBBBIHH", 0x10, 0x08 if dt.kind == "i" else 0x00, 0, 0, dt.itemsize, 0, 8 * dt.itemsize)
    if dt.kind == "f":
        n = dt.itemsize
        sign, exp_loc, exp_sz, man_sz, bias = {2: (15, 10, 5, 10, 15), 4: (31, 23, 8, 23, 127), 8: (63, 52, 11, 52, 1023)}[n]
        return struct.pack("<BBBBIHHBBBBI", 0x11, 0x20, sign, 0, n, 0, 8 * n, exp_loc, exp_sz, 0, man_sz, bias)
    raise Hdf5FormatError(f"cannot write dtype {dt}")


def _decode_dataspace(buf, at=0):
    ver, rank, flags = buf[at], buf[at + 1], buf[at + 2]
    if ver == 1:
        p = at + 8
    elif ver == 2:
        if buf[at + 3] == 2:
            return None                                                    # null dataspace
        p = at + 4
    else:
        raise Hdf5FormatError(f"dataspace message version {ver}")
    return tuple(struct.unpack_from("<Q", buf, p + 8 * i)[0] for i in range(rank))


def _encode_dataspace(shape):
    return struct.pack("<BBBB4x", 1, len(shape), 0, 0) + b"".join(struct.pack("<Q", int(d)) for d in shape)


def _pad8(n):
    return (n + 7) & ~7


def _decode_filters(m):
    """Filter pipeline message (0x000B) -> [(filter id, client data)]; versions 1 and 2."""
    ver, nf = m[0], m[1]
    p = 8 if ver == 1 else 2
    out = []
    for _ in range(nf):
        fid = struct.unpack_from("<H", m, p)[0]
        if ver == 1 or fid >= 256:
            name_len = struct.unpack_from("<H", m, p + 2)[0]
            flags, ncd = struct.unpack_from("<HH", m, p + 4)
            p += 8 + (_pad8(name_len) if ver == 1 else name_len)
        else:
            flags, ncd = struct.unpack_from("<HH", m, p + 2)
            p += 6
        cd = [struct.unpack_from("<I", m, p + 4 * i)[0] for i in range(ncd)]
        p += 4 * ncd + (4 if ver == 1 and ncd % 2 else 0)
        out.append((fid, cd))
    return tuple(out)


def _unfilter(fid, cd, raw, elem_size):
    if fid == 1:                                            # deflate
        import zlib
        return zlib.decompress(raw)
    if fid == 2:                                            # shuffle: byte planes back to elements
        n = len(raw) // elem_size
        a = np.frombuffer(raw, dtype=np.uint8, count=n * elem_size).reshape(elem_size, n)
        return a.T.tobytes() + raw[n * elem_size:]
    if fid == 3:                                            # fletcher32: four checksum bytes behind the data
        return raw[:-4]
    raise Hdf5FormatError(f"filter {fid} (only deflate, shuffle and fletcher32 are supported)")


# ----------------------------------------------------------------------------- reader
class _Node:
    def __init__(self, f, addr, name):
        self.f, self.addr, self.name = f, addr, name
        self._msgs = None

    def messages(self):
        if self._msgs is None:
            self._msgs = self.f._object_header(self.addr)
        return self._msgs

    @property
    def attrs(self):
        return {n: v for n, v in (self.f._attribute(m) for t, m in self.messages() if t == 0x000C)}

    def is_group(self):
        return any(t == 0x0011 for t, _ in self.messages())


class Hdf5Group(_Node):
    def _links(self):
        for t, m in self.messages():
            if t == 0x0011:
                btree, heap = struct.unpack_from("<QQ", m, 0)
                return dict(self.f._group_entries(btree, heap))
            if t in (0x0002, 0x0006):
                raise Hdf5FormatError("new-style groups (link info / link messages; files written with libver='latest')")
        return {}

    def keys(self):
        return sorted(self._links())

    def __contains__(self, name):
        try:
            self[name]
            return True
        except KeyError:
            return False

    def __getitem__(self, path):
        node = self
        for part in [p for p in path.split("/") if p]:
            if not isinstance(node, Hdf5Group):
                raise KeyError(path)
            links = node._links()
            if part not in links:
                raise KeyError(path)
            child = _Node(self.f, links[part], part)
            node = Hdf5Group(self.f, links[part], part) if child.is_group() else Hdf5Dataset(self.f, links[part], part)
        return node


class Hdf5Dataset(_Node):
    _filters = ()

    def _read_chunked(self, lay, shape, size, n):
        """Layout class 2: chunks of a fixed shape indexed by a version-1 B-tree whose keys carry the chunk's offset in the dataset."""
        if lay[0] != 3:
            raise Hdf5FormatError(f"chunked layout message version {lay[0]}")
        rank1 = lay[2]                                       # dataset rank + 1 (the last "dimension" is the element size)
        btree = struct.unpack_from("<Q", lay, 3)[0]
        cdims = [struct.unpack_from("<I", lay, 11 + 4 * i)[0] for i in range(rank1)]
        chunk_shape, rank = tuple(cdims[:-1]), rank1 - 1
        out = bytearray(n * size)
        arr = np.frombuffer(out, dtype=np.uint8).reshape(tuple(shape) + (size,)) if shape else None
        if btree == UNDEF:
            return bytes(out)
        for offsets, addr, nbytes, mask in self.f._chunk_entries(btree, rank1):
            raw = self.f._read(addr, nbytes)
            for k, (fid, cd) in enumerate(reversed(self._filters)):       # undo the pipeline back to front
                if mask & (1 << (len(self._filters) - 1 - k)):
                    continue                                          # this filter was skipped for this chunk
                raw = _unfilter(fid, cd, raw, size)
            chunk = np.frombuffer(raw, dtype=np.uint8, count=int(np.prod(chunk_shape)) * size).reshape(chunk_shape + (size,))
            sel = tuple(slice(o, min(o + c, s)) for o, c, s in zip(offsets, chunk_shape, shape))
            arr[sel] = chunk[tuple(slice(0, e.stop - e.start) for e in sel)]
        return bytes(out)

    def _meta(self):
        shape = dtype = layout = None
        for t, m in self.messages():
            if t == 0x0001:
                shape = _decode_dataspace(m)
            elif t == 0x0003:
                dtype = _decode_datatype(m)
            elif t == 0x0008:
                layout = m
            elif t == 0x000B:
                self._filters = _decode_filters(m)
        return shape, dtype, layout

    @property
    def shape(self):
        return self._meta()[0]

    def __array__(self, dtype=None, copy=None):
        a = self.read()
        return a.astype(dtype) if dtype is not None else a

    def read(self):
        shape, (kind, npdt, size, _), lay = self._meta()
        if kind != "num" and kind != "str":
            raise Hdf5FormatError("datasets of variable-length type")
        n = int(np.prod(shape)) if shape else 1
        ver = lay[0]
        if ver == 3:
            cls = lay[1]
            if cls == 1:
                addr, nbytes = struct.unpack_from("<QQ", lay, 2)
                raw = b"" if addr == UNDEF else self.f._read(addr, n * size)
            elif cls == 0:
                nbytes = struct.unpack_from("<H", lay, 2)[0]
                raw = bytes(lay[4:4 + nbytes])
            else:
                raw = self._read_chunked(lay, shape, size, n)
        elif ver in (1, 2):
            rank, cls = lay[1], lay[2]
            if cls == 1:
                addr = struct.unpack_from("<Q", lay, 8)[0]
                raw = self.f._read(addr, n * size)
            elif cls == 0:
                p = 8 + 4 * rank
                nbytes = struct.unpack_from("<I", lay, p)[0]
                raw = bytes(lay[p + 4:p + 4 + nbytes])
            else:
                raise Hdf5FormatError("chunked datasets")
        else:
            raise Hdf5FormatError(f"data layout message version {ver}")
        if len(raw) < n * size:
            raw = raw + b"\0" * (n * size - len(raw))                   # never-written contiguous data reads as the fill value 0
        return np.frombuffer(raw, dtype=npdt, count=n).reshape(shape or ()).copy()


class Hdf5File(Hdf5Group):
    def __init__(self, path_or_bytes):
        if isinstance(path_or_bytes, (bytes, bytearray, memoryview)):
            self.data = bytes(path_or_bytes)
        else:
            with open(path_or_bytes, "rb") as fh:
                self.data = fh.read()
        base = 0
        while base < len(self.data) and self.data[base:base + 8] != SIGNATURE:
            base = 512 if base == 0 else base * 2
        if base >= len(self.data):
            raise Hdf5FormatError("not an HDF5 file (signature not found)")
        ver = self.data[base + 8]
        if ver not in (0, 1):
            raise Hdf5FormatError(f"superblock version {ver} (files written with libver='latest')")
        if self.data[base + 13] != 8 or self.data[base + 14] != 8:
            raise Hdf5FormatError("offset / length sizes other than 8 bytes")
        p = base + 24 + (4 if ver == 1 else 0)
        self.base = struct.unpack_from("<Q", self.data, p)[0]
        root_entry = p + 32
        root_header = struct.unpack_from("<Q", self.data, root_entry + 8)[0]
        super().__init__(self, root_header, "/")

    def __enter__(self): return self
    def __exit__(self, *a): self.data = None

    # -- low level
    def _read(self, addr, n):
        a = self.base + addr
        if a + n > len(self.data):
            raise Hdf5FormatError("address beyond the end of the file")
        return self.data[a:a + n]

    def _object_header(self, addr):
        d, a = self.data, self.base + addr
        if d[a:a + 4] == b"OHDR":
            raise Hdf5FormatError("version-2 object headers (files written with libver='latest')")
        if d[a] != 1:
            raise Hdf5FormatError(f"object header version {d[a]}")
        nmsg = struct.unpack_from("<H", d, a + 2)[0]
        size = struct.unpack_from("<I", d, a + 8)[0]
        blocks, out = [(a + 16, size)], []
        while blocks and len(out) < nmsg:
            p, left = blocks.pop(0)
            end = p + left
            while p + 8 <= end and len(out) < nmsg:
                mtype, msize, _flags = struct.unpack_from("<HHB", d, p)
                body = d[p + 8:p + 8 + msize]
                if mtype == 0x0010:
                    off, length = struct.unpack_from("<QQ", body, 0)
                    blocks.append((self.base + off, length))
                out.append((mtype, body))
                p += 8 + _pad8(msize)
        return out

    def _heap_string(self, heap_addr, offset):
        h = self.base + heap_addr
        if self.data[h:h + 4] != b"HEAP":
            raise Hdf5FormatError("local heap signature")
        seg = struct.unpack_from("<Q", self.data, h + 24)[0]
        s = self.base + seg + offset
        e = self.data.index(b"\0", s)
        return self.data[s:e].decode("utf-8")

    def _group_entries(self, btree_addr, heap_addr):
        d, a = self.data, self.base + btree_addr
        if d[a:a + 4] == b"SNOD":
            n = struct.unpack_from("<H", d, a + 6)[0]
            for i in range(n):
                e = a + 8 + 40 * i
                name_off, hdr = struct.unpack_from("<QQ", d, e)
                yield self._heap_string(heap_addr, name_off), hdr
            return
        if d[a:a + 4] != b"TREE":
            raise Hdf5FormatError("B-tree node signature")
        if d[a + 4] != 0:
            raise Hdf5FormatError("B-tree node type (expected a group node)")
        used = struct.unpack_from("<H", d, a + 6)[0]
        p = a + 24                                                   # key 0
        for i in range(used):
            child = struct.unpack_from("<Q", d, p + 8)[0]
            yield from self._group_entries(child, heap_addr)
            p += 16

    def _chunk_entries(self, btree_addr, rank1):
        """(chunk offsets in the dataset, address, stored size, filter mask) of every chunk under a version-1 B-tree of type 1."""
        d, a = self.data, self.base + btree_addr
        if d[a:a + 4] != b"TREE" or d[a + 4] != 1:
            raise Hdf5FormatError("chunk B-tree node")
        level, used = d[a + 5], struct.unpack_from("<H", d, a + 6)[0]
        key_size = 8 + 8 * rank1
        p = a + 24
        for _ in range(used):
            nbytes, mask = struct.unpack_from("<II", d, p)
            offs = [struct.unpack_from("<Q", d, p + 8 + 8 * i)[0] for i in range(rank1 - 1)]
            child = struct.unpack_from("<Q", d, p + key_size)[0]
            if level == 0:
                yield offs, child, nbytes, mask
            else:
                yield from self._chunk_entries(child, rank1)
            p += key_size + 8

    def _global_heap_object(self, coll_addr, index):
        d, a = self.data, self.base + coll_addr
        if d[a:a + 4] != b"GCOL":
            raise Hdf5FormatError("global heap signature")
        size = struct.unpack_from("<Q", d, a + 8)[0]
        p, end = a + 16, a + size
        while p + 16 <= end:
            idx, _rc, osize = struct.unpack_from("<HH4xQ", d, p)
            if idx == index:
                return d[p + 16:p + 16 + osize]
            if idx == 0:
                break
            p += 16 + _pad8(osize)
        raise Hdf5FormatError("global heap object not found")

    def _attribute(self, m):
        ver = m[0]
        name_sz, dt_sz, ds_sz = struct.unpack_from("<HHH", m, 2)
        if ver == 1:
            p = 8
            name = bytes(m[p:p + name_sz]).split(b"\0")[0].decode("utf-8")
            p += _pad8(name_sz)
            dt_at = p
            p += _pad8(dt_sz)
            ds_at = p
            p += _pad8(ds_sz)
        elif ver in (2, 3):
            p = 8 if ver == 2 else 9
            name = bytes(m[p:p + name_sz]).split(b"\0")[0].decode("utf-8")
            p += name_sz
            dt_at = p
            p += dt_sz
            ds_at = p
            p += ds_sz
        else:
            raise Hdf5FormatError(f"attribute message version {ver}")
        kind, npdt, size, extra = _decode_datatype(m, dt_at)
        shape = _decode_dataspace(m, ds_at)
        n = int(np.prod(shape)) if shape else 1
        data = m[p:]
        if kind == "vlen_str":
            vals = []
            for i in range(n):
                length, coll, idx = struct.unpack_from("<IQI", data, 16 * i)
                vals.append(bytes(self._global_heap_object(coll, idx)[:length]).decode("utf-8") if length else "")
            return name, (vals[0] if not shape else np.array(vals, dtype=object).reshape(shape))
        arr = np.frombuffer(bytes(data[:n * size]), dtype=npdt, count=n)
        if kind == "str":
            arr = np.array([s.split(b"\0")[0] for s in arr.tolist()], dtype=object)
            return name, (arr[0] if not shape else arr.reshape(shape))
        return name, (arr[0] if not shape else arr.reshape(shape).copy())


# ----------------------------------------------------------------------------- writer
class Hdf5Writer:
    """Builds a file of the same subset: ``w = Hdf5Writer(); g = w.group("model_weights"); w.attr(g, "layer_names", [...]);
    w.dataset("model_weights/dense/kernel:0", array); w.save(path)``."""

    def __init__(self):
        self.tree = {"attrs": {}, "children": {}}

    def _node(self, path, create="group"):
        node = self.tree
        for part in [p for p in path.split("/") if p]:
            node = node["children"].setdefault(part, {"attrs": {}, "children": {}})
        return node

    def group(self, path):
        self._node(path)
        return path

    def dataset(self, path, array, chunks=None, compression=None, shuffle=False):
        """``chunks``: chunk shape (chunked layout); ``compression="gzip"`` and ``shuffle`` add the filters h5py would."""
        n = self._node(path)
        n["data"] = np.ascontiguousarray(array)
        if chunks is not None or compression or shuffle:
            n["chunks"] = tuple(chunks) if chunks is not None else tuple(max(1, d) for d in n["data"].shape)
            n["filters"] = ([2] if shuffle else []) + ([1] if compression else [])
        return path

    def attr(self, path, name, value):
        self._node(path)["attrs"][name] = value

    # -- serialisation
    def tobytes(self):
        out = bytearray(b"\0" * 96)                                   # superblock (56 bytes) + root symbol-table entry (40)

        def alloc(b, align=8):
            while len(out) % align:
                out.append(0)
            at = len(out)
            out.extend(b)
            return at

        def attr_message(name, value):
            if isinstance(value, str):
                raw = value.encode("utf-8")
                gcol = struct.pack("<4sB3xQ", b"GCOL", 1, 16 + 16 + _pad8(len(raw)) + 16)
                gcol += struct.pack("<HH4xQ", 1, 0, len(raw)) + raw + b"\0" * (_pad8(len(raw)) - len(raw))
                gcol += struct.pack("<HH4xQ", 0, 0, 0)                  # free-space object closes the collection
                coll = alloc(gcol)
                dt, ds, data = _encode_datatype("vlen_str"), struct.pack("<BBBB4x", 1, 0, 0, 0), struct.pack("<IQI", len(raw), coll, 1)
            else:
                arr = np.asarray(value)
                if arr.dtype.kind in "OU":
                    items = [s.encode("utf-8") if isinstance(s, str) else bytes(s) for s in arr.reshape(-1).tolist()]
                    arr = np.array(items, dtype=f"S{max(1, max((len(i) for i in items), default=1))}").reshape(arr.shape)
                dt, ds, data = _encode_datatype(arr.dtype), _encode_dataspace(arr.shape), np.ascontiguousarray(arr).tobytes()
            nm = name.encode("utf-8") + b"\0"
            body = struct.pack("<BBHHH", 1, 0, len(nm), len(dt), len(ds))
            for part in (nm, dt, ds):
                body += part + b"\0" * (_pad8(len(part)) - len(part))
            return 0x000C, body + data

        def header(messages):
            body = b""
            for mtype, m in messages:
                if len(m) > 0xFFF8:
                    raise Hdf5FormatError("header message larger than 64 KB (split the attribute as Keras does: name0, name1, ...)")
                body += struct.pack("<HHB3x", mtype, _pad8(len(m)), 0) + m + b"\0" * (_pad8(len(m)) - len(m))
            return alloc(struct.pack("<BBHII4x", 1, 0, len(messages), 1, len(body)) + body)

        def write_node(node):
            msgs = [attr_message(k, v) for k, v in node["attrs"].items()]
            if "data" in node and "chunks" in node:
                arr, cs, filters = node["data"], node["chunks"], node["filters"]
                esz, rank = arr.dtype.itemsize, arr.ndim
                entries = []
                import itertools
                import zlib
                for idx in itertools.product(*[range(0, max(s, 1), c) for s, c in zip(arr.shape, cs)]):
                    chunk = np.zeros(cs, dtype=arr.dtype)
                    sel = tuple(slice(o, min(o + c, s)) for o, c, s in zip(idx, cs, arr.shape))
                    chunk[tuple(slice(0, e.stop - e.start) for e in sel)] = arr[sel]
                    raw = chunk.tobytes()
                    for fid in filters:
                        if fid == 2:
                            raw = np.frombuffer(raw, dtype=np.uint8).reshape(-1, esz).T.tobytes()
                        elif fid == 1:
                            raw = zlib.compress(raw, 4)
                    entries.append((idx, alloc(raw), len(raw)))
                key = lambda offs, nbytes: struct.pack("<II", nbytes, 0) + b"".join(struct.pack("<Q", o) for o in offs) + struct.pack("<Q", 0)
                tree = struct.pack("<4sBBHQQ", b"TREE", 1, 0, len(entries), UNDEF, UNDEF)
                for idx, addr, nbytes in entries:
                    tree += key(idx, nbytes) + struct.pack("<Q", addr)
                tree += key(tuple(s for s in arr.shape), 0)                      # closing key: one past the last chunk
                btree = alloc(tree)
                layout = struct.pack("<BBBQ", 3, 2, rank + 1, btree) + b"".join(struct.pack("<I", c) for c in cs) + struct.pack("<I", esz)
                dmsgs = [(0x0001, _encode_dataspace(arr.shape)), (0x0003, _encode_datatype(arr.dtype)), (0x0008, layout)]
                if filters:
                    fm = struct.pack("<BB6x", 1, len(filters))
                    for fid in filters:
                        cd = [4] if fid == 1 else [esz]
                        fm += struct.pack("<HHHH", fid, 0, 1 if fid == 2 else 0, len(cd)) + b"".join(struct.pack("<I", c) for c in cd) + b"\0" * 4
                    dmsgs.append((0x000B, fm))
                return header(dmsgs + msgs), None
            if "data" in node:
                arr = node["data"]
                addr = alloc(arr.tobytes()) if arr.size else UNDEF
                layout = struct.pack("<BBQQ", 3, 1, addr, arr.nbytes)
                return header([(0x0001, _encode_dataspace(arr.shape)), (0x0003, _encode_datatype(arr.dtype)), (0x0008, layout)] + msgs), None
            names = sorted(node["children"])
            child_hdrs = {n: write_node(node["children"][n])[0] for n in names}
            heap_data = bytearray(b"\0" * 8)                          # offset 0: the empty name of the B-tree's first key
            offs = {}
            for n in names:
                offs[n] = len(heap_data)
                raw = n.encode("utf-8") + b"\0"
                heap_data.extend(raw + b"\0" * (_pad8(len(raw)) - len(raw)))
            seg = alloc(bytes(heap_data))
            heap = alloc(struct.pack("<4sB3xQQQ", b"HEAP", 0, len(heap_data), 1, seg))        # free-list head 1 = "no free block" (H5HL_FREE_NULL)
            snod = struct.pack("<4sBBH", b"SNOD", 1, 0, len(names))
            for n in names:
                snod += struct.pack("<QQII16x", offs[n], child_hdrs[n], 0, 0)
            snod += b"\0" * (40 * (2 * self.leaf_k - len(names)))
            snod_at = alloc(snod)
            tree = struct.pack("<4sBBHQQ", b"TREE", 0, 0, 1, UNDEF, UNDEF)
            tree += struct.pack("<QQQ", 0, snod_at, offs[names[-1]] if names else 0)
            tree += b"\0" * (16 * (2 * 16 - 1))                       # room for the unused keys / children of internal K = 16
            btree = alloc(tree)
            return header([(0x0011, struct.pack("<QQ", btree, heap))] + msgs), (btree, heap)

        def widest(node):
            return max([len(node["children"])] + [widest(c) for c in node["children"].values()])

        self.leaf_k = max(4, (widest(self.tree) + 1) // 2)
        root_hdr, (btree, heap) = write_node(self.tree)
        sb = SIGNATURE + struct.pack("<BBBBBBBBHHI", 0, 0, 0, 0, 0, 8, 8, 0, self.leaf_k, 16, 0)
        sb += struct.pack("<QQQQ", 0, UNDEF, len(out), UNDEF)
        sb += struct.pack("<QQII", 0, root_hdr, 1, 0) + struct.pack("<QQ", btree, heap)
        out[0:len(sb)] = sb
        return bytes(out)

    def save(self, path):
        with open(path, "wb") as f:
            f.write(self.tobytes())


# ----------------------------------------------------------------------------- Hdf5Archive
class Hdf5Archive:
    """The archive API the Keras importer of the reference is written against."""

    def __init__(self, path_or_bytes):
        self.file = Hdf5File(path_or_bytes)

    def _group(self, groups):
        node = self.file
        for g in groups:
            node = node[g]
        return node

    def hasAttribute(self, name, *groups):
        return name in self._group(groups).attrs

    def readAttributeAsString(self, name, *groups):
        v = self._group(groups).attrs[name]
        return v.decode("utf-8") if isinstance(v, bytes) else str(v)

    def readAttributeAsJson(self, name, *groups):
        import json
        return json.loads(self.readAttributeAsString(name, *groups))

    def readAttributeAsFixedLengthString(self, name, bufferSize, *groups):
        return self.readAttributeAsString(name, *groups)[:bufferSize]

    def readAttributeAsStringList(self, name, *groups):
        """A string-array attribute, joined over the ``name0, name1, ...`` pieces Keras splits long lists into."""
        attrs = self._group(groups).attrs
        parts = [attrs[name]] if name in attrs else []
        i = 0
        while f"{name}{i}" in attrs:
            parts.append(attrs[f"{name}{i}"])
            i += 1
        out = []
        for p in parts:
            for s in np.asarray(p, dtype=object).reshape(-1).tolist():
                out.append(s.decode("utf-8") if isinstance(s, bytes) else str(s))
        return out

    def readDataSet(self, datasetName, *groups):
        return self._group(groups)[datasetName].read()

    def getGroups(self, *groups):
        g = self._group(groups)
        return [k for k in g.keys() if isinstance(g[k], Hdf5Group)]

    def getDataSets(self, *groups):
        g = self._group(groups)
        return [k for k in g.keys() if isinstance(g[k], Hdf5Dataset)]

    def close(self):
        self.file = None

    def __enter__(self): return self
    def __exit__(self, *a): self.close()
