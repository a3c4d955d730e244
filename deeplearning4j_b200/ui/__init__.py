"""Training UI (``deeplearning4j-ui-parent``): ``StatsListener`` collecting per-iteration statistics, ``StatsStorage``
back-ends (in memory, sqlite file — the ``J7FileStatsStorage`` role), a ``RemoteUIStatsStorageRouter`` that POSTs
updates, and a small ``UIServer`` (stdlib HTTP) serving an overview page plus JSON endpoints for score, update ratios,
parameter / gradient histograms, memory and hardware information.

Statistics that need device data (mean magnitudes, histograms) are computed on the device in one pass over the flat
parameter / gradient buffers per layer and only the summaries are copied back, every ``listenerFrequency`` iterations."""
from __future__ import annotations

import http.server
import json
import os
import socket
import sqlite3
import threading
import time
import urllib.request
import uuid

import torch


class StatsUpdateConfiguration:
    def __init__(self, reportingFrequency=1, collectPerformanceStats=True, collectMemoryStats=True, collectLearningRates=True,
                 collectHistogramsParameters=True, collectHistogramsGradients=True, collectHistogramsUpdates=True, numHistogramBins=20,
                 collectMeanMagnitudesParameters=True, collectMeanMagnitudesGradients=True, collectMeanMagnitudesUpdates=True,
                 collectMeanParameters=True, collectStdevParameters=True):
        self.__dict__.update({k: v for k, v in locals().items() if k != "self"})


# ----------------------------------------------------------------------------- storage
class StatsStorageEvent:
    def __init__(self, kind, sessionID, typeID, workerID, timestamp):
        self.eventType, self.sessionID, self.typeID, self.workerID, self.timestamp = kind, sessionID, typeID, workerID, timestamp


class InMemoryStatsStorage:
    def __init__(self):
        self.static, self.updates, self.meta = {}, {}, {}
        self.listeners = []
        self.lock = threading.Lock()

    # -- router interface
    def putStorageMetaData(self, meta):
        self.meta[(meta["sessionID"], meta["typeID"])] = meta

    def putStaticInfo(self, rec):
        with self.lock:
            self.static[(rec["sessionID"], rec["typeID"], rec["workerID"])] = rec
        self._notify("PostStaticInfo", rec)

    def putUpdate(self, rec):
        with self.lock:
            self.updates.setdefault((rec["sessionID"], rec["typeID"], rec["workerID"]), []).append(rec)
        self._notify("PostUpdate", rec)

    def _notify(self, kind, rec):
        ev = StatsStorageEvent(kind, rec["sessionID"], rec["typeID"], rec["workerID"], rec["timestamp"])
        for l in self.listeners:
            l(ev)

    # -- query interface
    def registerStatsStorageListener(self, fn): self.listeners.append(fn)
    def deregisterStatsStorageListener(self, fn): self.listeners.remove(fn)
    def listSessionIDs(self): return sorted({k[0] for k in list(self.static) + list(self.updates)})
    def sessionExists(self, sid): return sid in self.listSessionIDs()
    def listTypeIDsForSession(self, sid): return sorted({k[1] for k in list(self.static) + list(self.updates) if k[0] == sid})
    def listWorkerIDsForSession(self, sid): return sorted({k[2] for k in list(self.static) + list(self.updates) if k[0] == sid})
    def getStaticInfo(self, sid, tid, wid): return self.static.get((sid, tid, wid))
    def getAllStaticInfos(self, sid, tid): return [v for k, v in self.static.items() if k[0] == sid and k[1] == tid]
    def getNumUpdateRecordsFor(self, sid, tid=None, wid=None):
        return sum(len(v) for k, v in self.updates.items() if k[0] == sid and (tid is None or k[1] == tid) and (wid is None or k[2] == wid))
    def getAllUpdatesAfter(self, sid, tid, wid=None, timestamp=0):
        out = []
        for k, v in self.updates.items():
            if k[0] == sid and k[1] == tid and (wid is None or k[2] == wid):
                out += [u for u in v if u["timestamp"] > timestamp]
        return sorted(out, key=lambda u: u["timestamp"])
    def getLatestUpdate(self, sid, tid, wid=None):
        u = self.getAllUpdatesAfter(sid, tid, wid, 0)
        return u[-1] if u else None
    def getLatestUpdateAllWorkers(self, sid, tid):
        return [v[-1] for k, v in self.updates.items() if k[0] == sid and k[1] == tid and v]
    def close(self): pass
    def isClosed(self): return False


class FileStatsStorage(InMemoryStatsStorage):
    """sqlite-backed storage: survives the process, can be re-opened by a UI server later."""

    def __init__(self, path):
        super().__init__()
        self.path = str(path)
        self.db = sqlite3.connect(self.path, check_same_thread=False)
        self.db.execute("CREATE TABLE IF NOT EXISTS static_info (sid TEXT, tid TEXT, wid TEXT, ts INTEGER, body TEXT, PRIMARY KEY (sid, tid, wid))")
        self.db.execute("CREATE TABLE IF NOT EXISTS updates (sid TEXT, tid TEXT, wid TEXT, ts INTEGER, body TEXT)")
        self.db.execute("CREATE INDEX IF NOT EXISTS upd_idx ON updates (sid, tid, ts)")
        self.db.commit()
        for sid, tid, wid, ts, body in self.db.execute("SELECT * FROM static_info"):
            self.static[(sid, tid, wid)] = json.loads(body)
        for sid, tid, wid, ts, body in self.db.execute("SELECT * FROM updates ORDER BY ts"):
            self.updates.setdefault((sid, tid, wid), []).append(json.loads(body))

    def putStaticInfo(self, rec):
        with self.lock:
            self.db.execute("INSERT OR REPLACE INTO static_info VALUES (?,?,?,?,?)", (rec["sessionID"], rec["typeID"], rec["workerID"], rec["timestamp"], json.dumps(rec)))
            self.db.commit()
        super().putStaticInfo(rec)

    def putUpdate(self, rec):
        with self.lock:
            self.db.execute("INSERT INTO updates VALUES (?,?,?,?,?)", (rec["sessionID"], rec["typeID"], rec["workerID"], rec["timestamp"], json.dumps(rec)))
            self.db.commit()
        super().putUpdate(rec)

    def close(self): self.db.close()


J7FileStatsStorage = FileStatsStorage
MapDBStatsStorage = FileStatsStorage


class RemoteUIStatsStorageRouter:
    """POSTs records to ``<address>/remoteReceive`` of a UIServer with remote listening enabled."""

    def __init__(self, address, maxRetries=3, retryDelayMs=200):
        self.url, self.maxRetries, self.retryDelayMs = address.rstrip("/") + "/remoteReceive", maxRetries, retryDelayMs
        self.failed = 0

    def _post(self, kind, rec):
        body = json.dumps({"type": kind, "record": rec}).encode()
        for attempt in range(self.maxRetries):
            try:
                req = urllib.request.Request(self.url, body, {"Content-Type": "application/json"})
                urllib.request.urlopen(req, timeout=5).read()
                return True
            except OSError:
                time.sleep(self.retryDelayMs / 1e3 * (attempt + 1))
        self.failed += 1
        return False

    def putStorageMetaData(self, meta): self._post("metadata", meta)
    def putStaticInfo(self, rec): self._post("static", rec)
    def putUpdate(self, rec): self._post("update", rec)


# ----------------------------------------------------------------------------- listener
class StatsListener:
    TYPE_ID = "StatsListener"

    def __init__(self, router, listenerFrequency=1, updateConfig=None, sessionID=None, workerID=None):
        self.router, self.frequency = router, max(int(listenerFrequency), 1)
        self.cfg = updateConfig or StatsUpdateConfiguration(reportingFrequency=listenerFrequency)
        self.sessionID = sessionID or str(uuid.uuid4())
        self.workerID = workerID or f"{socket.gethostname()}_{os.getpid()}"
        self._init_done = False
        self._last_time = None
        self._prev_params = None
        self._iter_since = 0
        self._examples_since = 0

    def getSessionID(self): return self.sessionID
    def getWorkerID(self): return self.workerID
    def getStorageRouter(self): return self.router

    def _static(self, model):
        layers = []
        owners = model._owners()
        for key, layer in owners:
            layers.append({"name": str(key), "type": type(layer).__name__, "nParams": sum(s.numel for s in layer.param_specs())})
        hw = {"hostname": socket.gethostname(), "nDevices": torch.cuda.device_count() if torch.cuda.is_available() else 0,
              "deviceNames": [torch.cuda.get_device_name(i) for i in range(torch.cuda.device_count())] if torch.cuda.is_available() else [],
              "deviceTotalMemory": [torch.cuda.get_device_properties(i).total_memory for i in range(torch.cuda.device_count())] if torch.cuda.is_available() else []}
        sw = {"torch": torch.__version__, "cuda": torch.version.cuda, "backend": "deeplearning4j_b200"}
        return {"sessionID": self.sessionID, "typeID": self.TYPE_ID, "workerID": self.workerID, "timestamp": int(time.time() * 1e3),
                "modelClass": type(model).__name__, "numLayers": len(owners), "numParams": int(model.numParams()), "layers": layers,
                "hardware": hw, "software": sw, "configJson": model.conf.toJson() if hasattr(model.conf, "toJson") else None}

    @staticmethod
    def _summaries(flat, entries, bins, hist, mean_mag, mean_std):
        out = {}
        for e in entries:
            if e.spec.kind == "state":
                continue
            seg = flat[e.offset:e.end].float()
            s = {}
            if mean_mag:
                s["meanMagnitude"] = float(seg.abs().mean())
            if mean_std:
                s["mean"], s["stdev"] = float(seg.mean()), float(seg.std(unbiased=False)) if seg.numel() > 1 else 0.0
            if hist:
                lo, hi = float(seg.min()), float(seg.max())
                if hi <= lo:
                    hi = lo + 1e-12
                s["histogram"] = {"min": lo, "max": hi, "counts": torch.histc(seg, bins=bins, min=lo, max=hi).long().tolist()}
            out[e.key] = s
        return out

    def iterationDone(self, model, iteration, epoch):
        if not self._init_done:
            self.router.putStorageMetaData({"sessionID": self.sessionID, "typeID": self.TYPE_ID, "workerID": self.workerID, "timestamp": int(time.time() * 1e3),
                                            "initTypeClass": "StatsInitializationReport", "updateTypeClass": "StatsReport"})
            self.router.putStaticInfo(self._static(model))
            self._init_done = True
            self._last_time = time.perf_counter()
        self._iter_since += 1
        self._examples_since += int(getattr(model, "_last_batch", 0) or 0)
        if iteration % self.frequency:
            return
        cfg = self.cfg
        now = time.perf_counter()
        rec = {"sessionID": self.sessionID, "typeID": self.TYPE_ID, "workerID": self.workerID, "timestamp": int(time.time() * 1e3),
               "iteration": iteration, "epoch": epoch, "score": float(model.score())}
        if cfg.collectPerformanceStats:
            dt = max(now - self._last_time, 1e-9)
            rec["performance"] = {"iterationsPerSecond": self._iter_since / dt, "examplesPerSecond": self._examples_since / dt,
                                  "totalRuntimeMs": int(dt * 1e3), "etlMs": float(getattr(model, "_last_etl_ms", 0.0) or 0.0)}
        if cfg.collectMemoryStats:
            mem = {}
            if model.flat_params.is_cuda:
                free, total = torch.cuda.mem_get_info(model.flat_params.device)
                mem = {"deviceCurrentBytes": [total - free], "deviceMaxBytes": [total], "allocatorReserved": torch.cuda.memory_reserved(model.flat_params.device)}
            try:
                import psutil
                vm = psutil.virtual_memory()
                mem.update({"jvmCurrentBytes": psutil.Process().memory_info().rss, "offHeapMaxBytes": vm.total})
            except ImportError:
                pass
            rec["memory"] = mem
        if cfg.collectLearningRates:
            lrs = {}
            upd = getattr(model, "updater", None)
            for b in getattr(upd, "blocks", []) or []:
                if b.config.hasLearningRate():
                    for e in b.entries:
                        lrs[e.key] = b.config.getLearningRate(iteration, epoch)
            rec["learningRates"] = lrs
        with torch.no_grad():
            rec["parameters"] = self._summaries(model.flat_params, model.entries, cfg.numHistogramBins, cfg.collectHistogramsParameters,
                                                cfg.collectMeanMagnitudesParameters, cfg.collectMeanParameters)
            rec["gradients"] = self._summaries(model.flat_grads, model.entries, cfg.numHistogramBins, cfg.collectHistogramsGradients,
                                               cfg.collectMeanMagnitudesGradients, False)
            if cfg.collectMeanMagnitudesUpdates or cfg.collectHistogramsUpdates:
                cur = model.flat_params.detach().clone()
                if self._prev_params is not None and self._prev_params.shape == cur.shape:
                    upd = self._summaries(cur - self._prev_params, model.entries, cfg.numHistogramBins, cfg.collectHistogramsUpdates,
                                          cfg.collectMeanMagnitudesUpdates, False)
                    rec["updates"] = upd
                    rec["updateRatios"] = {k: (v.get("meanMagnitude", 0.0) / max(rec["parameters"][k].get("meanMagnitude", 0.0), 1e-30))
                                           for k, v in upd.items() if "meanMagnitude" in v}
                self._prev_params = cur
        self.router.putUpdate(rec)
        self._last_time, self._iter_since, self._examples_since = time.perf_counter(), 0, 0

    def onEpochStart(self, model): pass
    def onEpochEnd(self, model): pass


# ----------------------------------------------------------------------------- server
_PAGE = """<!doctype html><html><head><meta charset="utf-8"><title>Training overview</title>
<style>body{font-family:sans-serif;margin:2em}table{border-collapse:collapse}td,th{border:1px solid #ccc;padding:4px 8px}</style></head>
<body><h2>Training overview</h2><div id="info"></div><svg id="chart" width="720" height="300" style="border:1px solid #ccc"></svg>
<h3>Layers</h3><table id="layers"></table>
<script>
async function refresh(){
 const s=await (await fetch('/train/sessions')).json(); if(!s.length){return}
 const sid=s[s.length-1];
 const o=await (await fetch('/train/overview?sid='+sid)).json();
 document.getElementById('info').textContent='session '+sid+' | iteration '+o.lastIteration+' | score '+o.lastScore+' | '+(o.examplesPerSecond||0).toFixed(1)+' examples/s';
 const pts=o.scores; const svg=document.getElementById('chart'); if(pts.length>1){
  const xs=pts.map(p=>p[0]),ys=pts.map(p=>p[1]); const x0=Math.min(...xs),x1=Math.max(...xs),y0=Math.min(...ys),y1=Math.max(...ys);
  svg.innerHTML='<polyline fill="none" stroke="#1f77b4" stroke-width="2" points="'+pts.map(p=>(20+680*(p[0]-x0)/Math.max(x1-x0,1e-9))+','+(280-260*(p[1]-y0)/Math.max(y1-y0,1e-9))).join(' ')+'"/>';}
 const m=await (await fetch('/train/model?sid='+sid)).json();
 document.getElementById('layers').innerHTML='<tr><th>layer</th><th>type</th><th>params</th></tr>'+m.layers.map(l=>'<tr><td>'+l.name+'</td><td>'+l.type+'</td><td>'+l.nParams+'</td></tr>').join('');
}
refresh(); setInterval(refresh,2000);
</script></body></html>"""


class UIServer:
    _instance = None

    def __init__(self, port=9000, host="127.0.0.1"):
        self.port, self.host = port, host
        self.storages = []
        self.remote = None
        self._httpd = None
        self._thread = None

    @classmethod
    def getInstance(cls, port=9000):
        if cls._instance is None:
            cls._instance = cls(port)
            cls._instance.start()
        return cls._instance

    def attach(self, storage):
        if storage not in self.storages:
            self.storages.append(storage)

    def detach(self, storage):
        if storage in self.storages:
            self.storages.remove(storage)

    def isAttached(self, storage): return storage in self.storages

    def registerModule(self, module):
        """Adds a module's routes (``ui/modules.py``: t-SNE, convolutional activations, SameDiff graph)."""
        self.__dict__.setdefault("modules", []).append(module)
        self.__dict__.setdefault("_routes", {}).update(module.routes())
        return self
    def getStatsStorageInstances(self): return list(self.storages)

    def enableRemoteListener(self, storage=None, attach=True):
        self.remote = storage or InMemoryStatsStorage()
        if attach:
            self.attach(self.remote)

    def disableRemoteListener(self): self.remote = None
    def getAddress(self): return f"http://{self.host}:{self.port}"
    def getPort(self): return self.port

    def _find(self, sid):
        for s in self.storages:
            if s.sessionExists(sid):
                return s
        return None

    def _json(self, path, query):
        sid = query.get("sid")
        if path == "/train/sessions":
            return sorted({x for s in self.storages for x in s.listSessionIDs()})
        st = self._find(sid) if sid else None
        if st is None:
            return {"error": "unknown session"}
        ups = st.getAllUpdatesAfter(sid, StatsListener.TYPE_ID, None, 0)
        if path == "/train/overview":
            last = ups[-1] if ups else {}
            return {"scores": [[u["iteration"], u["score"]] for u in ups], "lastIteration": last.get("iteration"), "lastScore": last.get("score"),
                    "examplesPerSecond": (last.get("performance") or {}).get("examplesPerSecond"), "memory": last.get("memory"),
                    "updateRatios": last.get("updateRatios")}
        if path == "/train/model":
            infos = st.getAllStaticInfos(sid, StatsListener.TYPE_ID)
            info = infos[0] if infos else {}
            last = ups[-1] if ups else {}
            return {"layers": info.get("layers", []), "numParams": info.get("numParams"), "parameters": last.get("parameters"),
                    "gradients": last.get("gradients"), "updates": last.get("updates"), "learningRates": last.get("learningRates")}
        if path == "/train/system":
            infos = st.getAllStaticInfos(sid, StatsListener.TYPE_ID)
            return {"hardware": [i.get("hardware") for i in infos], "software": [i.get("software") for i in infos],
                    "memory": [[u["timestamp"], u.get("memory")] for u in ups]}
        return {"error": "unknown endpoint"}

    def start(self):
        server = self

        class H(http.server.BaseHTTPRequestHandler):
            def log_message(self, *a): pass

            def _send(self, code, body, ctype):
                self.send_response(code)
                self.send_header("Content-Type", ctype)
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def do_GET(self):
                from urllib.parse import parse_qs, urlparse
                u = urlparse(self.path)
                q = {k: v[0] for k, v in parse_qs(u.query).items()}
                if u.path in ("/", "/train", "/train/overview.html"):
                    return self._send(200, _PAGE.encode(), "text/html; charset=utf-8")
                route = server.__dict__.get("_routes", {}).get(("GET", u.path))
                if route is not None:
                    code, ctype, body = route(q, b"")
                    return self._send(code, body, ctype)
                return self._send(200, json.dumps(server._json(u.path, q)).encode(), "application/json")

            def do_POST(self):
                from urllib.parse import parse_qs, urlparse
                n = int(self.headers.get("Content-Length", 0))
                raw = self.rfile.read(n)
                u = urlparse(self.path)
                route = server.__dict__.get("_routes", {}).get(("POST", u.path))
                if route is not None:
                    code, ctype, out = route({k: v[0] for k, v in parse_qs(u.query).items()}, raw)
                    return self._send(code, out, ctype)
                body = json.loads(raw or b"{}")
                if self.path != "/remoteReceive" or server.remote is None:
                    return self._send(403, b'{"error": "remote listener disabled"}', "application/json")
                kind, rec = body.get("type"), body.get("record")
                {"metadata": server.remote.putStorageMetaData, "static": server.remote.putStaticInfo, "update": server.remote.putUpdate}[kind](rec)
                return self._send(200, b'{"status": "ok"}', "application/json")

        self._httpd = http.server.ThreadingHTTPServer((self.host, self.port), H)
        self.port = self._httpd.server_address[1]
        self._thread = threading.Thread(target=self._httpd.serve_forever, daemon=True)
        self._thread.start()
        return self

    def stop(self):
        if self._httpd is not None:
            self._httpd.shutdown()
            self._httpd.server_close()
            self._httpd = None
        if UIServer._instance is self:
            UIServer._instance = None


from .modules import (ChartHistogram, ChartHorizontalBar, ChartLine, ChartScatter, ChartStackedArea, ChartTimeline, Component,  # noqa: E402,F401
                      ComponentDiv, ComponentTable, ComponentText, ConvolutionalIterationListener, ConvolutionalListenerModule,
                      DecoratorAccordion, SameDiffModule, StaticPageUtil, TsneModule, UIModule, decode_stats, encode_stats)
