"""NVTX ranges around ops, layers and training phases, so that a profiler timeline (or ``ncu --nvtx --nvtx-include``) can be read by
layer / op name instead of by kernel name.  Off by default: ``DL4J_NVTX=1`` or ``nvtx.enable()`` switches it on; when off, ``range``
is a shared no-op context and costs one attribute test.  The reference's counterparts are its per-op profiling hooks
(``OpProfiler``, ``ProfilingListener``); the NVTX form is what the CUDA tools consume directly."""
from __future__ import annotations

import contextlib
import os

import torch

_on = os.environ.get("DL4J_NVTX", "0") not in ("", "0")
_null = contextlib.nullcontext()
_log = None            # list of (event, name) when recording for tests, else None


def enable(on=True):
    global _on
    _on = bool(on)


def enabled():
    return _on


def record(log):
    """Also append ("push" | "pop", name) to ``log`` (a list); ``None`` stops it.  Used by tests on machines without a GPU."""
    global _log
    _log = log


def push(name):
    if _log is not None:
        _log.append(("push", name))
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)


def pop():
    if _log is not None:
        _log.append(("pop", None))
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_pop()


class _Range:
    __slots__ = ("name",)

    def __init__(self, name): self.name = name
    def __enter__(self): push(self.name)
    def __exit__(self, *a): pop()


def range(name):
    return _Range(name) if _on else _null


class NvtxListener:
    """SameDiff listener: one range per executed op, named ``<opName>:<node name>``."""

    def __getattr__(self, name):                    # every other listener hook is a no-op
        if name.startswith("_"):
            raise AttributeError(name)
        return lambda *a, **k: None

    def isActive(self, operation=None): return True
    def preOpExecution(self, sd, op): push(f"{op.opName}:{op.name}")
    def opExecution(self, sd, op, outputs): pop()
