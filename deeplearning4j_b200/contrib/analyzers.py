"""Developer tools in the spirit of the reference's ``contrib/``: a profiler-output analyzer (``unified-profiler-analyzer``), a
native-source dependency analyzer (``cpp-dependency-analyzer``) and an op-registry report (``op-registry-updater``)."""
from __future__ import annotations

import collections
import csv
import os
import re


# ------------------------------------------------------------------------------------------------------ profiler output
def kernel_shares(csv_path, metric="gpu__time_duration.sum", top=None, strip_templates=True):
    """Aggregates a launch list written by ``ncu --csv --metrics gpu__time_duration.sum`` into (kernel, launches, total, share) rows
    sorted by total time; lines that are not CSV records (profiler banners) are skipped."""
    with open(csv_path, newline="") as f:
        lines = [l for l in f if not l.startswith("==")]
    rows = list(csv.DictReader(lines))
    agg = collections.OrderedDict()
    unit = None
    for r in rows:
        if r.get("Metric Name") not in (None, metric):
            continue
        name = r["Kernel Name"]
        if strip_templates:
            name = re.sub(r"\(.*", "", re.sub(r"<.*", "", name)).replace("void ", "").strip()
        v = float(r["Metric Value"].replace(",", ""))
        unit = r.get("Metric Unit", unit)
        a = agg.setdefault(name, [0, 0.0])
        a[0] += 1
        a[1] += v
    scale = {"ns": 1e-6, "us": 1e-3, "usecond": 1e-3, "nsecond": 1e-6, "ms": 1.0, "msecond": 1.0}.get(unit or "ns", 1e-6)
    total = sum(v for _, v in agg.values()) or 1.0
    out = [{"kernel": k, "launches": n, "ms": v * scale, "share": v / total} for k, (n, v) in agg.items()]
    out.sort(key=lambda r: -r["ms"])
    return out[:top] if top else out


def shares_markdown(rows):
    lines = ["| share | time | launches | kernel |", "|---|---|---|---|"]
    lines += [f"| {100 * r['share']:.1f} % | {r['ms']:.3f} ms | {r['launches']} | {r['kernel']} |" for r in rows]
    return "\n".join(lines)


def step_boundaries(csv_path, marker="fused_update"):
    """Indices of the launches whose kernel name contains ``marker`` (one per training step): slices of the list between two of
    them are whole steps."""
    with open(csv_path, newline="") as f:
        rows = list(csv.DictReader(l for l in f if not l.startswith("==")))
    return [i for i, r in enumerate(rows) if marker in r["Kernel Name"]]


# ------------------------------------------------------------------------------------------------------ native sources
_INC = re.compile(r'^\s*#\s*include\s*"([^"]+)"', re.M)
_KERNEL = re.compile(r"__global__\s+void(?:\s+__launch_bounds__\([^)]*\))?\s+(\w+)")
_API = re.compile(r"DL4J_API\s+[\w\s\*]+?\s+\**(\w+)\s*\(")


def native_dependencies(src_dir):
    """Per source file of the native library: local headers it includes (transitively), kernels it defines, C entry points it exports."""
    files = {f: open(os.path.join(src_dir, f), errors="replace").read() for f in sorted(os.listdir(src_dir)) if f.endswith((".cu", ".cuh", ".h"))}
    direct = {f: [i for i in _INC.findall(t) if i in files] for f, t in files.items()}

    def closure(f, seen=None):
        seen = set() if seen is None else seen
        for i in direct.get(f, []):
            if i not in seen:
                seen.add(i)
                closure(i, seen)
        return seen
    return {f: {"includes": sorted(closure(f)), "kernels": _KERNEL.findall(t), "exports": _API.findall(t)} for f, t in files.items()}


def rebuild_set(src_dir, changed):
    """Translation units that must be recompiled when ``changed`` (a file name) is touched."""
    deps = native_dependencies(src_dir)
    return sorted(f for f, d in deps.items() if f.endswith(".cu") and (f == changed or changed in d["includes"]))


# ------------------------------------------------------------------------------------------------------ op registry
def registry_report():
    """Counts per group, names without a reference counterpart and reference names without an implementation."""
    from ..ops import registry
    from ..ops.reference_ops import REFERENCE_OP_NAMES as REFERENCE_OPS
    registry.load_all()
    groups = collections.Counter(registry.get(n).group for n in registry.names())
    ref = set(REFERENCE_OPS)
    return {"registered": len(registry.names()), "groups": dict(groups), "missing": sorted(n for n in ref if not registry.has(n)),
            "extra": sorted(n for n in registry.names() if n not in ref and "." not in n)[:2000]}
