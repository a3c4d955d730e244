"""Op-execution log and regression diff.

Parity: ``contrib/nd4j-log-analyzer`` (a Java agent that records every executed op with its inputs / outputs into an H2 database and
compares two runs to find the first op whose results diverge) and ``contrib/unified-profiler-analyzer`` (aggregating timing
events).  Here a SameDiff listener records, per executed op, its name, type, input / output shapes and dtypes, a checksum and
simple statistics of every output and the wall time, into a sqlite file; ``OpLogAnalyzer.compare`` lines two logs up by op name
and reports the first divergence and all ops whose output statistics differ by more than a tolerance, ``summary`` aggregates time
by op type.
"""
from __future__ import annotations

import json
import sqlite3
import time
import zlib

import torch


def _stats(t):
    if not isinstance(t, torch.Tensor) or t.numel() == 0:
        return {"shape": [], "dtype": "", "crc": 0, "mean": 0.0, "absmax": 0.0, "nan": 0}
    f = t.detach().float()
    c = t.detach().contiguous().cpu().reshape(-1)
    raw = c.view(torch.uint8).numpy().tobytes() if t.dtype != torch.bool else c.numpy().tobytes()
    return {"shape": list(t.shape), "dtype": str(t.dtype), "crc": zlib.crc32(raw), "mean": float(f.mean()), "absmax": float(f.abs().max()),
            "nan": int(torch.isnan(f).sum())}


class OpLogListener:
    """SameDiff listener writing one row per executed op (attach with ``sd.addListeners(OpLogListener(path))``)."""

    def __init__(self, path, run="run"):
        self.db = sqlite3.connect(path)
        self.db.execute("CREATE TABLE IF NOT EXISTS ops (run TEXT, seq INTEGER, name TEXT, op TEXT, inputs TEXT, outputs TEXT, ms REAL)")
        self.run, self.seq, self._t0 = run, 0, None

    def preOpExecution(self, sd, node):
        self._t0 = time.perf_counter()

    def opExecution(self, sd, node, outs):
        ms = (time.perf_counter() - self._t0) * 1e3 if self._t0 is not None else 0.0
        ins = [{"name": i} for i in node.inputs if i is not None]
        self.db.execute("INSERT INTO ops VALUES (?, ?, ?, ?, ?, ?, ?)",
                        (self.run, self.seq, node.name, node.opName, json.dumps(ins), json.dumps([_stats(o) for o in outs]), ms))
        self.seq += 1

    def close(self):
        self.db.commit()
        self.db.close()


class OpLogAnalyzer:
    @staticmethod
    def load(path, run=None):
        db = sqlite3.connect(path)
        q = "SELECT seq, name, op, outputs, ms FROM ops" + (" WHERE run = ?" if run else "") + " ORDER BY seq"
        rows = db.execute(q, (run,) if run else ()).fetchall()
        db.close()
        return [{"seq": s, "name": n, "op": o, "outputs": json.loads(out), "ms": ms} for s, n, o, out, ms in rows]

    @staticmethod
    def compare(path_a, path_b, run_a=None, run_b=None, rtol=1e-4):
        a, b = OpLogAnalyzer.load(path_a, run_a), OpLogAnalyzer.load(path_b, run_b)
        by_b = {r["name"]: r for r in b}
        diverged, missing = [], []
        for r in a:
            o = by_b.get(r["name"])
            if o is None:
                missing.append(r["name"])
                continue
            for k, (x, y) in enumerate(zip(r["outputs"], o["outputs"])):
                if x["shape"] != y["shape"] or x["dtype"] != y["dtype"]:
                    diverged.append({"name": r["name"], "op": r["op"], "output": k, "reason": "shape/dtype", "a": x, "b": y})
                elif x["crc"] != y["crc"]:
                    scale = max(abs(x["absmax"]), abs(y["absmax"]), 1e-12)
                    if abs(x["mean"] - y["mean"]) > rtol * scale or abs(x["absmax"] - y["absmax"]) > rtol * scale or x["nan"] != y["nan"]:
                        diverged.append({"name": r["name"], "op": r["op"], "output": k, "reason": "values", "a": x, "b": y})
        return {"first_divergence": diverged[0] if diverged else None, "diverged": diverged, "missing_in_b": missing,
                "extra_in_b": [r["name"] for r in b if r["name"] not in {x["name"] for x in a}]}

    @staticmethod
    def summary(path, run=None, top=20):
        agg = {}
        for r in OpLogAnalyzer.load(path, run):
            e = agg.setdefault(r["op"], [0, 0.0])
            e[0] += 1
            e[1] += r["ms"]
        return sorted(((op, n, ms) for op, (n, ms) in agg.items()), key=lambda x: -x[2])[:top]
