"""SameDiff <-> FlatGraph (``graph.fbs``) mapping.

Parity: ``autodiff/samediff/serde/FlatBuffersMapper.java`` and ``SameDiff.asFlatBuffers`` /
``fromFlatBuffers`` (``autodiff/samediff/SameDiff.java:6218-6760``).  Layout choices kept from the
reference: variables get id pairs (node id, output index) with leaf variables numbered first; ops are
``CUSTOM`` nodes whose ``opNum`` is the op-name hash; op arguments travel as ``FlatProperties``;
``trainingConfig`` is the JSON string; updater state is one ``UpdaterState`` table per parameter with
named state arrays; arrays are ``FlatArray`` with plain shape, c-order little-endian bytes.
"""
from __future__ import annotations

import numpy as np
import torch

from ...nd.dtype import DataType
from ...ops import registry
from . import flatbuffers as fb

# DataType ids are the libnd4j ids, which are also the values of the schema's DType enum
_DT_TO_FB = {d: int(d) for d in DataType if int(d) <= 52}
_FB_TO_DT = {v: k for k, v in _DT_TO_FB.items()}

_STATE_KEYS = {"Sgd": [], "NoOp": [], "Nesterovs": ["V"], "Adam": ["M", "V"], "AdaMax": ["M", "V"], "Nadam": ["M", "V"],
               "AMSGrad": ["M", "V", "V_HAT"], "AdaBelief": ["M", "S"], "AdaGrad": ["grad"], "RmsProp": ["G"],
               "AdaDelta": ["msg", "msdx"]}


# ----------------------------------------------------------------------------- arrays
def flat_array(t: torch.Tensor) -> dict:
    t = t.detach()
    dt = DataType.from_torch(t.dtype)
    tc = t.contiguous().cpu()
    if tc.dtype == torch.bfloat16:
        raw = tc.view(torch.int16).numpy()
    elif tc.dtype == torch.bool:
        raw = tc.to(torch.uint8).numpy()
    else:
        raw = tc.numpy()
    return {"shape": list(t.shape), "buffer": memoryview(np.ascontiguousarray(raw)).cast("B"), "dtype": _DT_TO_FB[dt], "byteOrder": 0}


class Utf8Array(list):
    """A string array (``DType.UTF8``) read from a FlatArray: a list of ``str`` with the array's shape kept beside it.  Strings do
    not live in tensors; ops that take them (``Assert`` messages, ``print_variable``) receive this object."""

    def __init__(self, items, shape=()):
        super().__init__(items)
        self.shape = tuple(shape)


def _shape_info(vec):
    """``FlatArray.shape`` in the reference's classic form is the full shapeInfo vector
    ``[rank, shape.., stride.., extras, elementWiseStride, order]`` (``libnd4j/include/graph/impl/FlatUtils.cpp:37-62``): length
    ``2 rank + 4`` with the order character ('c' = 99, 'f' = 102) last.  Returns ``(shape, order, empty)`` or None when ``vec`` is
    a plain shape (what this framework and ``SameDiffSerializer`` write)."""
    n = len(vec)
    if n < 4:
        return None
    rank = int(vec[0])
    if rank < 0 or n != 2 * rank + 4 or int(vec[-1]) not in (99, 102):
        return None
    shape = [int(s) for s in vec[1:1 + rank]]
    extras = int(vec[2 * rank + 1])
    return shape, ("f" if int(vec[-1]) == 102 else "c"), bool(extras & 8)        # ARRAY_EMPTY = 8 (array/ArrayOptions.h)


def _decode_utf8(buf, shape):
    """libnd4j string buffer: ``int64 offsets[n + 1]`` followed by the bytes (``array/impl/NDArrayFactory.cpp`` string_*)."""
    n = int(np.prod(shape)) if shape else 1
    raw = bytes(buf)
    for order in (">", "<"):
        if len(raw) < 8 * (n + 1):
            break
        offs = np.frombuffer(raw, dtype=order + "i8", count=n + 1)
        data = raw[8 * (n + 1):]
        if offs[0] == 0 and all(0 <= int(offs[i]) <= int(offs[i + 1]) <= len(data) for i in range(n)):
            return Utf8Array([data[int(offs[i]):int(offs[i + 1])].decode("utf-8", "replace") for i in range(n)], shape)
    return Utf8Array([raw.decode("utf-8", "replace")], shape)


def from_flat_array(a: dict, device=None):
    dt = _FB_TO_DT[a["dtype"]]
    vec = [int(s) for s in (a["shape"] if a["shape"] is not None else [])]
    info = _shape_info(vec)
    shape, forder, empty = (vec, "c", False) if info is None else info
    buf = a["buffer"]
    if dt.name in ("UTF8", "UTF16", "UTF32"):
        return _decode_utf8(buf if buf is not None else b"", shape)
    tdt = dt.to_torch()
    n = int(np.prod(shape)) if shape else 1
    if empty or buf is None or len(buf) == 0:
        if empty and not shape:
            shape = [0]
        return torch.zeros(shape, dtype=tdt, device=device)
    order = ">" if a.get("byteOrder", 0) == 1 else "<"
    if tdt == torch.bfloat16:
        t = torch.from_numpy(np.frombuffer(buf, dtype=order + "i2", count=n).astype("<i2")).view(torch.bfloat16)
    elif tdt == torch.bool:
        t = torch.from_numpy(np.frombuffer(buf, dtype=np.uint8, count=n).copy()).to(torch.bool)
    else:
        npdt = np.dtype(torch.empty(0, dtype=tdt).numpy().dtype).newbyteorder(order)
        t = torch.from_numpy(np.frombuffer(buf, dtype=npdt, count=n).astype(npdt.newbyteorder("=")))
    if forder == "f" and len(shape) > 1:
        t = t.reshape(list(reversed(shape))).permute(*reversed(range(len(shape)))).contiguous()
    else:
        t = t.reshape(shape)
    return t.to(device) if device is not None else t


# ----------------------------------------------------------------------------- op arguments
def _flatten(v):
    arr = np.asarray(v)
    return arr.reshape(-1).tolist(), list(arr.shape)


def _property(name, v) -> dict:
    p = {"name": name}
    if isinstance(v, torch.Tensor):
        p["a"] = [flat_array(v)]
    elif isinstance(v, bool):
        p["b"] = [v]
    elif isinstance(v, DataType):
        p["i"] = [int(v)]
        p["s"] = ["DataType"]
    elif isinstance(v, (int, np.integer)):
        p["l"] = [int(v)]
    elif isinstance(v, (float, np.floating)):
        p["d"] = [float(v)]
    elif isinstance(v, str):
        p["s"] = [v]
    elif isinstance(v, (list, tuple)):
        if len(v) == 0:
            p["l"], p["shape"] = [], [0]
        elif all(isinstance(x, str) for x in v):
            p["s"], p["shape"] = list(v), [len(v)]
        elif all(isinstance(x, torch.Tensor) for x in v):
            p["a"], p["shape"] = [flat_array(x) for x in v], [len(v)]
        else:
            flat, shape = _flatten(v)
            if all(isinstance(x, bool) for x in flat):
                p["b"] = flat
            elif all(isinstance(x, (int, np.integer)) and not isinstance(x, bool) for x in flat):
                p["l"] = [int(x) for x in flat]
            else:
                p["d"] = [float(x) for x in flat]
            p["shape"] = shape
    else:
        raise TypeError(f"op argument {name!r} of type {type(v).__name__} cannot be stored in a FlatGraph")
    return p


def _from_property(p: dict):
    shape = p.get("shape")
    shape = None if shape is None else [int(s) for s in shape]
    s, a = p.get("s"), p.get("a")
    if p.get("i") is not None and len(p["i"]) and s and s[0] == "DataType":
        return DataType(int(p["i"][0]))
    for key, conv in (("b", bool), ("l", int), ("d", float), ("i", int)):
        vals = p.get(key)
        if vals is not None and (len(vals) or shape == [0]):
            vals = [conv(x) for x in vals]
            if shape is None:
                return vals[0]
            return np.asarray(vals, dtype=object).reshape(shape).tolist() if len(shape) > 1 else vals
    if a:
        arrs = [from_flat_array(x) for x in a]
        return arrs[0] if shape is None else arrs
    if s is not None and len(s):
        return s[0] if shape is None else list(s)
    return [] if shape == [0] else None



# ----------------------------------------------------------------------------- nodes written by the reference
_LOGIC_OPS = {0: "while", 10: "scope", 20: "conditional", 30: "switch", 40: "return", 60: "merge", 70: "loop_cond",
              80: "next_iteration", 90: "exit", 100: "enter"}          # libnd4j/include/graph/execution/LogicExecutor + sd::logic ids
_FAMILY = {"PAIRWISE": "PAIRWISE_TRANSFORM", "REDUCE_3": "REDUCE3", "SUMMARYSTATS": "SUMMARY_STATS"}
_TF_LIST_OPS = {"tensorarrayv3": "tf_list_create", "tensorarraywritev3": "tf_list_write", "tensorarrayreadv3": "tf_list_read",
                "tensorarraygatherv3": "tf_list_gather", "tensorarrayscatterv3": "tf_list_scatter", "tensorarraysplitv3": "tf_list_split",
                "tensorarraysizev3": "tf_list_size", "tensorarrayconcatv3": "tf_list_concat", "tensorarrayclosev3": "noop",
                "stridedslice": "strided_slice"}


def _resolve_op_name(fn, op_type):
    """Op name of a FlatNode: its ``opName`` when present, else CUSTOM ops by hash, LOGIC ops by their fixed numbers and every
    legacy family through the ``(op type, opNum)`` table (``LegacyOpMapper.java:71``)."""
    from .legacy_ops import LEGACY_OPS
    name = fn["opName"]
    num = int(fn["opNum"])
    if op_type == "LOGIC":
        return _LOGIC_OPS.get(num, name or f"logic_{num}")
    if op_type not in ("CUSTOM", "UDF", "GRAPH"):
        fam = LEGACY_OPS.get(_FAMILY.get(op_type, op_type), {})
        if num in fam:
            legacy = fam[num][1]
            if not name or not registry.has(name):
                return legacy
    if name:
        return name
    return registry.name_for_hash(num)


def _reference_style(fn) -> bool:
    """True for nodes whose arguments are positional (iArgs / tArgs / bArgs / dimensions / scalar), as the reference writes them;
    this framework stores keyword arguments as properties and never fills those vectors."""
    for k in ("extraInteger", "extraParams", "extraBools", "dimensions"):
        v = fn[k]
        if v is not None and len(v):
            return True
    if fn["scalar"] is not None:
        return True
    props = {p["name"] for p in (fn["properties"] or [])}
    return bool(props & {"bArguments", "inplaceCall", "dimensionz", "passThrough"})


def _reference_args(fn, op_name, op_type):
    from ...ops import argschema
    scalar = from_flat_array(fn["scalar"]) if fn["scalar"] is not None else None
    args = argschema.kwargs_for(op_name, op_type, fn["extraInteger"], fn["extraParams"], fn["extraBools"], fn["dimensions"], scalar,
                                fn["extraTypes"])
    for p in fn["properties"] or []:
        if p["name"] in ("frameName", "isConstant"):
            v = _from_property(p)
            if isinstance(v, (list, tuple)):
                v = v[0] if len(v) else None
            if v is not None:
                args[p["name"]] = v
    if op_type in ("SCALAR", "SCALAR_BOOL") and scalar is not None and op_name not in argschema.SCHEMAS:
        args["_scalar"] = scalar
    return args


def _adapt_reference_op(op_name, ins, args, sd):
    """Last step of the import of a reference node: TensorFlow-style list ops get their executable names, legacy scalar ops get
    their scalar as a second (constant) input, reductions drop a dimension input that only says "all dimensions"."""
    op_name = _TF_LIST_OPS.get(op_name, op_name)
    if op_name == "pad" and len(ins) == 3 and ins[2] is not None:
        pv = sd.arrays.get(ins[2])                    # PadV2: the fill value arrives as a third (constant) input
        if isinstance(pv, torch.Tensor):
            args["padValue"] = float(pv.reshape(-1)[0])
            ins = ins[:2]
    sc = args.pop("_scalar", None)
    if sc is not None:
        c = sd.constant(None, sc)
        ins = list(ins[:1]) + [c.name] + list(ins[1:])
    if (op_name.startswith("reduce_") or op_name in ("all", "any", "argmax", "argmin")) and len(ins) == 2 and ins[1] is not None:
        arr = sd.arrays.get(ins[1])
        if arr is not None and isinstance(arr, torch.Tensor):
            dims = [int(d) for d in arr.reshape(-1).tolist()]
            ins = ins[:1]
            if dims and "dimensions" not in args and not (len(dims) == 1 and dims[0] == 2147483647):
                args["dimensions"] = dims
    return op_name, ins, args


def _order_ops(sd):
    """Nodes of a file may come in any order; the plain session executes ``sd.ops`` front to back, so sort them topologically
    (graphs with loops keep their cycles -- those run on the frame-aware executor, which does not depend on the order)."""
    produced_by = {o: n for n in sd.ops for o in n.outputs}
    done, order, state = set(), [], {}

    def visit(n):
        stack = [(n, iter([produced_by.get(i) for i in n.inputs if i is not None]))]
        state[id(n)] = 1
        while stack:
            node, it = stack[-1]
            nxt = next(it, "end")
            if nxt == "end":
                stack.pop()
                state[id(node)] = 2
                order.append(node)
                continue
            if nxt is None or state.get(id(nxt)):
                continue                                   # leaf input, finished, or a back edge of a loop
            state[id(nxt)] = 1
            stack.append((nxt, iter([produced_by.get(i) for i in nxt.inputs if i is not None])))
    for n in list(sd.ops):
        if not state.get(id(n)):
            visit(n)
    sd.ops[:] = order


# ----------------------------------------------------------------------------- graph
def _updater_states(sd):
    st = getattr(sd, "_training", None)
    if st is None or st.updater is None or st.updater.state is None or st.updater.state.numel() == 0:
        return []
    out = []
    state = st.updater.state
    for b in st.updater.blocks:
        keys = _STATE_KEYS.get(type(b.config).__name__, [f"S{i}" for i in range(b.config.STATE_MULT)])
        n = b.numel
        for e in b.entries:
            rel = e.offset - b.start
            vals = [state[b.state_offset + k * n + rel: b.state_offset + k * n + rel + e.spec.numel].view(e.spec.shape)
                    for k in range(len(keys))]
            if keys:
                out.append({"paramName": e.spec.name, "updaterStateKeys": list(keys), "updaterStateValues": [flat_array(v) for v in vals]})
    return out


def to_flatbuffers(sd, saveUpdaterState=True) -> bytes:
    from ..core import VariableType
    ids, variables = {}, []
    counter = 0
    leaf_types = (VariableType.VARIABLE, VariableType.CONSTANT, VariableType.PLACEHOLDER)
    for name, v in sd.variables.items():
        if v.variableType in leaf_types:
            counter += 1
            ids[name] = (counter, 0)
    op_ids = {}
    for op in sd.ops:
        counter += 1
        op_ids[op.name] = counter
        for k, o in enumerate(op.outputs):
            ids[o] = (counter, k)
    for name, v in sd.variables.items():
        if name not in ids:                                    # ARRAY variable without a producer (dangling)
            counter += 1
            ids[name] = (counter, 0)
        fv = {"id": {"first": ids[name][0], "second": ids[name][1]}, "name": name, "variabletype": fb.VARTYPE.get(v.variableType, 2),
              "device": -1}
        arr = sd.arrays.get(name) if v.variableType in (VariableType.VARIABLE, VariableType.CONSTANT) else None
        if arr is not None:
            fv["ndarray"] = flat_array(arr)
            fv["dtype"] = _DT_TO_FB[DataType.from_torch(arr.dtype)]
            fv["shape"] = list(arr.shape)
        else:
            if v._dtype is not None:
                fv["dtype"] = _DT_TO_FB.get(v._dtype, 0)
            if v._shape is not None:
                fv["shape"] = [int(s) if s is not None else -1 for s in v._shape]
        variables.append(fv)
    nodes = []
    for op in sd.ops:
        node = {"id": op_ids[op.name], "name": op.name, "opType": fb.OPTYPE["CUSTOM"], "opNum": registry.op_hash(op.opName),
                "opName": op.opName, "device": -1, "outputNames": list(op.outputs),
                "inputPaired": [{"first": ids[i][0], "second": ids[i][1]} if i is not None else {"first": -1, "second": -1}
                                for i in op.inputs],
                "properties": [_property(k, v) for k, v in op.args.items()]}
        if op.controlDeps:
            node["controlDeps"] = list(op.controlDeps)
        nodes.append(node)
    g = {"id": 119, "variables": variables, "nodes": nodes,
         "outputs": [{"first": ids[o][0], "second": ids[o][1]} for o in sd.outputs() if o in ids],
         "configuration": {"id": 119, "outputMode": 4, "direction": 0},
         "placeholders": sd.inputs(), "lossVariables": list(sd.lossVariables)}
    if sd.trainingConfig is not None:
        g["trainingConfig"] = sd.trainingConfig.toJson()
    if saveUpdaterState:
        us = _updater_states(sd)
        if us:
            g["updaterState"] = us
    if sd.metadata:
        g["metadataKeys"] = [str(k) for k in sd.metadata]
        g["metadataValues"] = [str(v) for v in sd.metadata.values()]
    return fb.encode("FlatGraph", g)


def from_flatbuffers(buf, loadUpdaterState=True):
    from ..core import SameDiff, SameDiffOp, SDVariable
    from ..training import TrainingConfig, _ensure_state
    g = fb.decode("FlatGraph", buf)
    sd = SameDiff()
    vt_names = {v: k for k, v in fb.VARTYPE.items()}
    by_id = {}
    for fv in g["variables"] or []:
        name = fv["name"]
        vtype = vt_names.get(fv["variabletype"], "ARRAY")
        dt = _FB_TO_DT.get(fv["dtype"]) if fv["dtype"] else None
        shape = None if fv["shape"] is None else tuple(int(s) for s in fv["shape"])
        var = SDVariable(sd, name, vtype, dt, shape)
        sd.variables[name] = var
        if fv["ndarray"] is not None:
            sd.arrays[name] = from_flat_array(fv["ndarray"])
        if fv["id"] is not None:
            by_id[(fv["id"]["first"], fv["id"]["second"])] = name
    optype_names = {v: k for k, v in fb.OPTYPE.items()}
    for fn in g["nodes"] or []:
        pairs = fn["inputPaired"]
        if pairs is not None and len(pairs):
            ins = [by_id.get((p["first"], p["second"])) if p["first"] >= 0 else None for p in pairs]
        else:
            ins = [by_id.get((int(i), 0)) for i in (fn["input"] if fn["input"] is not None else [])]
        op_type = optype_names.get(fn["opType"], "CUSTOM")
        op_name = _resolve_op_name(fn, op_type)
        if _reference_style(fn):
            args = _reference_args(fn, op_name, op_type)
        else:
            args = {p["name"]: _from_property(p) for p in (fn["properties"] or [])}
        outs = list(fn["outputNames"] or [])
        if not outs:
            # files older than the ``outputNames`` field: outputs are the variables registered under (node id, k)
            k = 0
            while (fn["id"], k) in by_id:
                outs.append(by_id[(fn["id"], k)])
                k += 1
        op_name, ins, args = _adapt_reference_op(op_name, ins, args, sd)
        node = SameDiffOp(fn["name"] or f"node_{fn['id']}", op_name, ins, outs, args, list(fn["controlDeps"] or []))
        sd.ops.append(node)
        for o in node.outputs:
            sd._producer[o] = node
    _order_ops(sd)
    sd.lossVariables = list(g["lossVariables"] or [])
    if g["trainingConfig"]:
        sd.trainingConfig = TrainingConfig.fromJson(g["trainingConfig"])
    if g["metadataKeys"]:
        sd.metadata = dict(zip(g["metadataKeys"], g["metadataValues"] or []))
    if loadUpdaterState and g["updaterState"] and sd.trainingConfig is not None:
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
                    dst.copy_(from_flat_array(fa).reshape(-1).to(dst.dtype))
    return sd
