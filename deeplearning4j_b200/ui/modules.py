"""UI modules beyond the training pages, UI components and the binary stats record
(``deeplearning4j-vertx/.../ui/module/{tsne,convolutional,SameDiffModule}``, ``deeplearning4j-ui-components``,
``deeplearning4j-ui-model/.../stats/sbe``).

A module contributes routes to ``UIServer`` (``UIServer.registerModule``): ``routes()`` maps (method, path) to a function of
(query dict, body bytes) that returns (status, content type, payload bytes).
"""
from __future__ import annotations

import io
import json
import struct
import time

import numpy as np
import torch


# ------------------------------------------------------------------------------------------------------ modules
class UIModule:
    def routes(self): return {}
    def onAttach(self, storage): return None
    def onDetach(self, storage): return None


def _j(obj, status=200):
    return status, "application/json", json.dumps(obj).encode()


class TsneModule(UIModule):
    """Upload and serve 2-D embedding coordinates with labels (``TsneModule.java``: ``/tsne/upload``, ``/tsne/sessions``,
    ``/tsne/coords/:sid``).  The upload format is the reference's text form, one point per line: ``x,y,label``."""

    def __init__(self): self.sessions = {}

    def setCoordinates(self, sessionId, coords, labels=None):
        c = np.asarray(coords.cpu() if isinstance(coords, torch.Tensor) else coords, dtype=np.float64)
        labels = [str(l) for l in labels] if labels is not None else [str(i) for i in range(len(c))]
        self.sessions[str(sessionId)] = [f"{x:.6g},{y:.6g},{l}" for (x, y), l in zip(c[:, :2], labels)]

    def routes(self):
        def upload(q, body):
            lines = [l for l in body.decode("utf-8", "replace").splitlines() if l.strip()]
            for l in lines:
                if len(l.split(",")) < 3:
                    return _j({"error": f"expected x,y,label per line, got {l[:40]!r}"}, 400)
            self.sessions[q.get("sid", "UploadedFile")] = lines
            return _j({"status": "ok", "points": len(lines)})
        return {("POST", "/tsne/upload"): upload,
                ("GET", "/tsne/sessions"): lambda q, b: _j(sorted(self.sessions)),
                ("GET", "/tsne/coords"): lambda q, b: _j(self.sessions.get(q.get("sid", "UploadedFile"), []))}


def _grid_image(acts, pad=1):
    """[C, H, W] activations -> one uint8 image with the channels tiled on a near-square grid, each scaled to 0..255."""
    a = acts.detach().float().cpu()
    c, h, w = a.shape
    cols = int(np.ceil(np.sqrt(c)))
    rows = int(np.ceil(c / cols))
    lo, hi = a.amin((1, 2), keepdim=True), a.amax((1, 2), keepdim=True)
    a = ((a - lo) / (hi - lo).clamp_min(1e-12) * 255.0).to(torch.uint8)
    out = torch.zeros(rows * (h + pad) + pad, cols * (w + pad) + pad, dtype=torch.uint8)
    for i in range(c):
        r, k = divmod(i, cols)
        out[pad + r * (h + pad):pad + r * (h + pad) + h, pad + k * (w + pad):pad + k * (w + pad) + w] = a[i]
    return out.numpy()


def _png(gray):
    """Minimal PNG encoder for an 8-bit grey image (no Pillow needed to serve activations)."""
    import zlib
    h, w = gray.shape
    raw = b"".join(b"\x00" + gray[r].tobytes() for r in range(h))

    def chunk(tag, data):
        return struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)
    return b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, 0, 0, 0, 0)) + chunk(b"IDAT", zlib.compress(raw, 6)) + chunk(b"IEND", b"")


class ConvolutionalIterationListener:
    """Every ``frequency`` iterations renders the activations of the convolutional layers for the first example of the last
    batch into one image per layer and hands them to a ``ConvolutionalListenerModule`` (``ConvolutionalIterationListener.java``)."""

    def __init__(self, module, frequency=10, sessionId=None):
        self.module, self.freq, self.sid = module, max(int(frequency), 1), sessionId or f"conv_{int(time.time() * 1000)}"

    def iterationDone(self, model, iteration, epoch=0):
        if iteration % self.freq:
            return
        x = getattr(model, "_last_input", None)
        if x is None:
            return
        with torch.no_grad():
            acts = model.feedForward(x[:1] if isinstance(x, torch.Tensor) else x, False)
        acts = acts.values() if isinstance(acts, dict) else acts
        images = []
        for a in acts:
            t = a.t if hasattr(a, "t") and not isinstance(a, torch.Tensor) else a
            if isinstance(t, torch.Tensor) and t.dim() == 4:
                images.append(_grid_image(t[0]))
        if images:
            self.module.setImages(self.sid, iteration, images)

    def onEpochStart(self, model): pass
    def onEpochEnd(self, model): pass


class ConvolutionalListenerModule(UIModule):
    """``/activations`` page data: the latest rendered activation images (``ConvolutionalListenerModule.java``)."""

    def __init__(self): self.latest = {}

    def setImages(self, sid, iteration, images): self.latest[sid] = (int(iteration), [_png(i) for i in images])

    def routes(self):
        def data(q, b):
            sid = q.get("sid") or (sorted(self.latest)[-1] if self.latest else None)
            if sid not in self.latest:
                return _j({"error": "no activations yet"}, 404)
            it, imgs = self.latest[sid]
            k = int(q.get("layer", 0))
            if k < 0 or k >= len(imgs):
                return _j({"error": f"layer {k} of {len(imgs)}"}, 404)
            return 200, "image/png", imgs[k]
        return {("GET", "/activations/data"): data,
                ("GET", "/activations/info"): lambda q, b: _j({s: {"iteration": v[0], "layers": len(v[1])} for s, v in self.latest.items()})}


class SameDiffModule(UIModule):
    """Graph structure of a SameDiff instance for the graph page (``SameDiffModule.java`` reads a UI log file; here the instance
    or a ``.fb`` file is given directly): variables with type / shape / data type, ops with inputs and outputs."""

    def __init__(self): self.graphs = {}

    def setGraph(self, name, sd):
        if isinstance(sd, (str, bytes)):
            from ..samediff.core import SameDiff
            sd = SameDiff.fromFlatFile(sd) if isinstance(sd, str) else SameDiff.fromFlatBuffers(sd)
        vs = []
        for n, v in sd.variables.items():
            arr = sd.arrays.get(n)
            vs.append({"name": n, "type": str(getattr(v, "variableType", "")).split(".")[-1],
                       "shape": list(arr.shape) if arr is not None else None, "dataType": str(arr.dtype).replace("torch.", "") if arr is not None else None})
        ops = [{"name": o.name, "op": o.opName, "inputs": [i for i in o.inputs if i is not None], "outputs": list(o.outputs),
                "args": {k: (v if isinstance(v, (int, float, str, bool, list)) else str(v)) for k, v in o.args.items()}} for o in sd.ops]
        self.graphs[name] = {"variables": vs, "ops": ops}

    def routes(self):
        return {("GET", "/samediff/graphs"): lambda q, b: _j(sorted(self.graphs)),
                ("GET", "/samediff/graph"): lambda q, b: _j(self.graphs.get(q.get("name", ""), {"error": "unknown graph"}))}


# ------------------------------------------------------------------------------------------------------ components
class Component:
    """Serialisable page component (``deeplearning4j-ui-components``): ``toJson`` gives the reference's
    ``{"componentType": ..., ...}`` wrapper objects; ``StaticPageUtil.renderHTML`` writes a standalone page."""
    componentType = "Component"

    def __init__(self, **kw): self.kw = kw
    def toDict(self): return {"componentType": self.componentType, **{k: v for k, v in self.kw.items() if v is not None}}
    def toJson(self): return json.dumps(self.toDict())


class _ChartBuilderMixin:
    @classmethod
    def Builder(cls, title=None, style=None): return _ChartBuilder(cls, title, style)


class _ChartBuilder:
    def __init__(self, cls, title, style): self.cls, self.kw = cls, {"title": title, "style": style, "series": []}
    def addSeries(self, name, x, y=None):
        s = {"name": name, "x": [float(v) for v in x]}
        if y is not None:
            s["y"] = [float(v) for v in y]
        self.kw["series"].append(s)
        return self
    def addBin(self, lower, upper, value):
        self.kw.setdefault("bins", []).append({"lower": float(lower), "upper": float(upper), "y": float(value)})
        return self
    def setXMin(self, v): self.kw["xmin"] = float(v); return self
    def setXMax(self, v): self.kw["xmax"] = float(v); return self
    def setYMin(self, v): self.kw["ymin"] = float(v); return self
    def setYMax(self, v): self.kw["ymax"] = float(v); return self
    def build(self): return self.cls(**self.kw)


class ChartLine(Component, _ChartBuilderMixin): componentType = "ChartLine"
class ChartScatter(Component, _ChartBuilderMixin): componentType = "ChartScatter"
class ChartHistogram(Component, _ChartBuilderMixin): componentType = "ChartHistogram"
class ChartStackedArea(Component, _ChartBuilderMixin): componentType = "ChartStackedArea"
class ChartHorizontalBar(Component, _ChartBuilderMixin): componentType = "ChartHorizontalBar"
class ChartTimeline(Component, _ChartBuilderMixin): componentType = "ChartTimeline"


class ComponentText(Component):
    componentType = "ComponentText"
    def __init__(self, text, style=None): super().__init__(text=str(text), style=style)


class ComponentTable(Component):
    componentType = "ComponentTable"
    def __init__(self, header=None, content=None, style=None):
        super().__init__(header=list(header) if header else None, content=[[str(c) for c in r] for r in (content or [])], style=style)


class ComponentDiv(Component):
    componentType = "ComponentDiv"
    def __init__(self, style=None, *components): super().__init__(style=style, components=[c.toDict() for c in components])


class DecoratorAccordion(Component):
    componentType = "DecoratorAccordion"
    def __init__(self, title, defaultCollapsed=True, *components):
        super().__init__(title=title, defaultCollapsed=bool(defaultCollapsed), innerComponents=[c.toDict() for c in components])


class StaticPageUtil:
    @staticmethod
    def renderHTML(*components):
        """A standalone HTML page: the components as JSON plus a small renderer (tables, text, line / scatter charts on canvas)."""
        comps = [c.toDict() for c in (components[0] if len(components) == 1 and isinstance(components[0], (list, tuple)) else components)]
        return ("<!DOCTYPE html><html><head><meta charset='utf-8'><title>DL4J UI components</title></head><body><div id='root'></div><script>"
                "const comps=" + json.dumps(comps) + ";"
                "function el(t,p,s){const e=document.createElement(t);if(s)e.textContent=s;p.appendChild(e);return e}"
                "function draw(c,p){if(c.componentType=='ComponentText')el('p',p,c.text);"
                "else if(c.componentType=='ComponentTable'){const t=el('table',p);t.border=1;if(c.header){const r=el('tr',t);c.header.forEach(h=>el('th',r,h))}"
                "(c.content||[]).forEach(row=>{const r=el('tr',t);row.forEach(v=>el('td',r,v))})}"
                "else if(c.componentType=='ComponentDiv'||c.componentType=='DecoratorAccordion'){const d=el('div',p);if(c.title)el('h3',d,c.title);"
                "(c.components||c.innerComponents||[]).forEach(x=>draw(x,d))}"
                "else{if(c.title)el('h3',p,c.title);const cv=el('canvas',p);cv.width=640;cv.height=320;const g=cv.getContext('2d');"
                "let xs=[],ys=[];(c.series||[]).forEach(s=>{xs=xs.concat(s.x);ys=ys.concat(s.y||[])});(c.bins||[]).forEach(b=>{xs.push(b.lower,b.upper);ys.push(b.y,0)});"
                "const x0=Math.min(...xs),x1=Math.max(...xs),y0=Math.min(...ys),y1=Math.max(...ys);"
                "const X=v=>20+600*(v-x0)/((x1-x0)||1),Y=v=>300-280*(v-y0)/((y1-y0)||1);"
                "(c.series||[]).forEach((s,k)=>{g.strokeStyle=g.fillStyle=['#c00','#06c','#090','#f80'][k%4];g.beginPath();"
                "s.x.forEach((v,i)=>{if(c.componentType=='ChartScatter')g.fillRect(X(v)-2,Y(s.y[i])-2,4,4);else if(i)g.lineTo(X(v),Y(s.y[i]));else g.moveTo(X(v),Y(s.y[i]))});g.stroke()});"
                "(c.bins||[]).forEach(b=>{g.fillStyle='#06c';g.fillRect(X(b.lower),Y(b.y),X(b.upper)-X(b.lower)-1,Y(y0)-Y(b.y))})}}"
                "comps.forEach(c=>draw(c,document.getElementById('root')));</script></body></html>")

    @staticmethod
    def saveHTMLFile(path, *components):
        with open(path, "w", encoding="utf-8") as f:
            f.write(StaticPageUtil.renderHTML(*components))


# ------------------------------------------------------------------------------------------------------ binary stats records
_MAGIC = b"DL4JSTAT"


def encode_stats(rec: dict) -> bytes:
    """A stats record (what ``StatsListener`` hands to a storage router) as one compact binary message.  The reference encodes its
    reports with generated Simple-Binary-Encoding codecs (``ui/model/stats/sbe/*``); this layout follows the same idea, fixed
    header fields first and variable-length groups after them, without claiming byte compatibility:

    ``magic[8] | version u16 | timestamp i64 | iteration i32 | epoch i32 | score f64 | n_groups u16`` then per group
    ``name_len u16 | name | kind u8 (0 scalar map, 1 histogram map, 2 json) | payload_len u32 | payload``; scalar maps are
    ``count u32`` x (``key_len u16 | key | f64``); histogram maps ``count u32`` x (``key_len u16 | key | min f64 | max f64 | nbins u32 | u32[nbins]``)."""
    def s(b): return struct.pack("<H", len(b)) + b
    head = _MAGIC + struct.pack("<Hqiid", 1, int(rec.get("timestamp", 0)), int(rec.get("iteration", -1)), int(rec.get("epoch", -1)),
                                float(rec.get("score", float("nan")) if rec.get("score") is not None else float("nan")))
    groups = []
    for name, val in rec.items():
        if name in ("timestamp", "iteration", "epoch", "score"):
            continue
        if isinstance(val, dict) and val and all(isinstance(v, (int, float)) and not isinstance(v, bool) for v in val.values()):
            payload = struct.pack("<I", len(val)) + b"".join(s(k.encode()) + struct.pack("<d", float(v)) for k, v in val.items())
            kind = 0
        elif isinstance(val, dict) and val and all(isinstance(v, dict) and {"min", "max", "counts"} <= set(v) for v in val.values()):
            payload = struct.pack("<I", len(val)) + b"".join(
                s(k.encode()) + struct.pack("<ddI", float(v["min"]), float(v["max"]), len(v["counts"])) + struct.pack(f"<{len(v['counts'])}I", *[int(c) for c in v["counts"]])
                for k, v in val.items())
            kind = 1
        else:
            payload, kind = json.dumps(val).encode(), 2
        groups.append(s(name.encode()) + struct.pack("<BI", kind, len(payload)) + payload)
    return head + struct.pack("<H", len(groups)) + b"".join(groups)


def decode_stats(buf: bytes) -> dict:
    if buf[:8] != _MAGIC:
        raise ValueError("not a stats record")
    ver, ts, it, ep, score = struct.unpack_from("<Hqiid", buf, 8)
    if ver != 1:
        raise ValueError(f"unknown stats record version {ver}")
    pos = 8 + struct.calcsize("<Hqiid")
    rec = {"timestamp": ts, "iteration": it, "epoch": ep, "score": None if score != score else score}
    n, = struct.unpack_from("<H", buf, pos)
    pos += 2

    def rs():
        nonlocal pos
        l, = struct.unpack_from("<H", buf, pos)
        pos += 2
        v = buf[pos:pos + l].decode()
        pos += l
        return v
    for _ in range(n):
        name = rs()
        kind, plen = struct.unpack_from("<BI", buf, pos)
        pos += 5
        end = pos + plen
        if kind == 2:
            rec[name] = json.loads(buf[pos:end].decode())
        else:
            cnt, = struct.unpack_from("<I", buf, pos)
            pos += 4
            d = {}
            for _ in range(cnt):
                k = rs()
                if kind == 0:
                    d[k], = struct.unpack_from("<d", buf, pos)
                    pos += 8
                else:
                    mn, mx, nb = struct.unpack_from("<ddI", buf, pos)
                    pos += 20
                    d[k] = {"min": mn, "max": mx, "counts": list(struct.unpack_from(f"<{nb}I", buf, pos))}
                    pos += 4 * nb
            rec[name] = d
        pos = end
    return rec
