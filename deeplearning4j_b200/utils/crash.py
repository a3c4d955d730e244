"""``CrashReportingUtil`` (``deeplearning4j-nn/.../util/CrashReportingUtil.java``): when training runs out of memory a text dump with
the memory state, the network's configuration summary and the per-layer parameter / activation sizes is written next to the
working directory (or where ``crashDumpOutputDirectory`` points), and the exception is re-raised."""
from __future__ import annotations

import os
import platform
import time

import torch

_ENABLED = os.environ.get("DL4J_CRASH_DUMP_ENABLED", "true").lower() not in ("0", "false", "no")
_DIR = os.environ.get("DL4J_CRASH_DUMP_OUTPUT_DIRECTORY")


def _fmt(n):
    for unit in ("B", "KB", "MB", "GB", "TB"):
        if abs(n) < 1024 or unit == "TB":
            return f"{n:.2f} {unit}" if unit != "B" else f"{int(n)} B"
        n /= 1024.0


class CrashReportingUtil:
    @staticmethod
    def crashDumpsEnabled(enabled): globals().__setitem__("_ENABLED", bool(enabled))
    @staticmethod
    def crashDumpOutputDirectory(path): globals().__setitem__("_DIR", None if path is None else os.fspath(path))
    @staticmethod
    def isOutOfMemory(e): return isinstance(e, (MemoryError, torch.cuda.OutOfMemoryError)) or "out of memory" in str(e).lower()

    @staticmethod
    def generateMemoryStatus(net, minibatch=None, exception=None):
        L = ["Deeplearning4j OOM Exception Encountered for " + type(net).__name__, f"Timestamp: {time.strftime('%Y-%m-%d %H:%M:%S')}",
             f"Thread: {os.getpid()}", ""]
        if exception is not None:
            L += ["========== Exception ==========", f"{type(exception).__name__}: {exception}", ""]
        L += ["========== Memory Information ==========", f"Host: {platform.node()} ({platform.platform()})", f"torch {torch.__version__}"]
        if torch.cuda.is_available():
            for d in range(torch.cuda.device_count()):
                free, total = torch.cuda.mem_get_info(d)
                st = torch.cuda.memory_stats(d)
                L.append(f"Device {d}: {torch.cuda.get_device_name(d)}  total {_fmt(total)}  free {_fmt(free)}  allocated "
                         f"{_fmt(st.get('allocated_bytes.all.current', 0))} (peak {_fmt(st.get('allocated_bytes.all.peak', 0))})  reserved "
                         f"{_fmt(st.get('reserved_bytes.all.current', 0))}  allocation retries {st.get('num_alloc_retries', 0)}  OOMs {st.get('num_ooms', 0)}")
        else:
            L.append("No CUDA device")
        try:
            from .workspace import BasicWorkspaceManager
            wss = BasicWorkspaceManager.instance().getAllWorkspacesForCurrentThread() if hasattr(BasicWorkspaceManager, "instance") else []
            L += ["", "========== Workspace Information ==========", f"Workspaces of this thread: {len(wss)}"]
            L += [f"  {w.getId()}: size {_fmt(w.getCurrentSize())}, spilled {_fmt(w.getSpilledSize())}, generation {w.getGenerationId()}" for w in wss]
        except Exception as e:          # noqa: BLE001
            L.append(f"(workspace information unavailable: {e})")
        L += ["", "========== Network Information =========="]
        n_params = net.numParams() if hasattr(net, "numParams") else 0
        fp = getattr(net, "flat_params", None)
        esz = fp.element_size() if fp is not None else 4
        L.append(f"Network # Parameters: {n_params}  ({_fmt(n_params * esz)} as {str(fp.dtype).replace('torch.', '') if fp is not None else 'float32'})")
        upd = getattr(net, "updater", None) or (net.getUpdater() if hasattr(net, "getUpdater") else None)
        state = getattr(upd, "state", None)
        if state is not None:
            L.append(f"Updater state: {state.numel()} values ({_fmt(state.numel() * state.element_size())})")
        sh = getattr(net, "flat_shadow", None)
        if sh is not None:
            L.append(f"Low-precision parameter shadow: {_fmt(sh.numel() * sh.element_size())}")
        if minibatch is not None:
            L.append(f"Minibatch size: {minibatch}")
        L += ["", "========== Layer Information =========="]
        for e in getattr(net, "entries", []) or []:
            spec = e.spec
            L.append(f"  {getattr(e, 'name', '?'):40s} {str(tuple(getattr(spec, 'shape', ()))):24s} {e.end - e.offset:>12d} values  kind {getattr(spec, 'kind', '')}")
        try:
            L += ["", "========== Configuration ==========", net.summary() if hasattr(net, "summary") else ""]
        except Exception as e:          # noqa: BLE001
            L.append(f"(summary unavailable: {e})")
        return "\n".join(L) + "\n"

    @staticmethod
    def writeMemoryCrashDump(net, exception, minibatch=None):
        """Writes ``dl4j-memory-crash-dump-<millis>_<pid>.txt``; returns its path (None when dumps are switched off)."""
        if not _ENABLED:
            return None
        d = _DIR or os.getcwd()
        os.makedirs(d, exist_ok=True)
        path = os.path.join(d, f"dl4j-memory-crash-dump-{int(time.time() * 1000)}_{os.getpid()}.txt")
        with open(path, "w", encoding="utf-8") as f:
            f.write(CrashReportingUtil.generateMemoryStatus(net, minibatch, exception))
        return path


def guard_fit(fn):
    """Decorator for ``fit``: an out-of-memory error leaves a crash dump behind before it propagates
    (``MultiLayerNetwork.java:1697-1699``)."""
    def wrapped(self, *a, **kw):
        try:
            return fn(self, *a, **kw)
        except (MemoryError, RuntimeError) as e:
            if CrashReportingUtil.isOutOfMemory(e):
                try:
                    p = CrashReportingUtil.writeMemoryCrashDump(self, e)
                    if p:
                        e.args = (f"{e.args[0] if e.args else e} [memory crash dump written to {p}]",) + tuple(e.args[1:])
                except Exception:       # noqa: BLE001  (the dump must never mask the original error)
                    pass
            raise
    wrapped.__name__, wrapped.__doc__ = fn.__name__, fn.__doc__
    return wrapped
