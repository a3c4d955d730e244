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


def from_flat_array(a: dict, device=None) -> torch.Tensor:
    dt = _FB_TO_DT[a["dtype"]]
    shape = [int(s) for s in (a["shape"] if a["shape"] is not None else [])]
    tdt = dt.to_torch()
    n = int(np.prod(shape)) if shape else 1
    buf = a["buffer"]
    if buf is None or len(buf) == 0:
        return torch.zeros(shape, dtype=tdt, device=device)
    order = ">" if a.get("byteOrder", 0) == 1 else "<"
    if tdt == torch.bfloat16:
        t = torch.from_numpy(np.frombuffer(buf, dtype=order + "i2", count=n).astype("<i2")).view(torch.bfloat16)
    elif tdt == torch.bool:
        t = torch.from_numpy(np.frombuffer(buf, dtype=np.uint8, count=n).copy()).to(torch.bool)
    else:
        npdt = np.dtype(torch.empty(0, dtype=tdt).numpy().dtype).newbyteorder(order)
        t = torch.from_numpy(np.frombuffer(buf, dtype=npdt, count=n).astype(npdt.newbyteorder("=")))
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
    for fn in g["nodes"] or []:
        ins = [by_id.get((p["first"], p["second"])) if p["first"] >= 0 else None for p in (fn["inputPaired"] or [])]
        args = {p["name"]: _from_property(p) for p in (fn["properties"] or [])}
        op_name = fn["opName"] or registry.name_for_hash(fn["opNum"])
        node = SameDiffOp(fn["name"], op_name, ins, list(fn["outputNames"] or []), args, list(fn["controlDeps"] or []))
        sd.ops.append(node)
        for o in node.outputs:
            sd._producer[o] = node
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
