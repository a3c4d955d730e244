"""``python4j``: run Python snippets with typed inputs / outputs (``PythonExecutioner``, ``PythonVariables``, ``PythonGIL``,
``PythonContextManager``, ``PythonTypes``, numpy <-> INDArray bridge).

The reference embeds CPython in the JVM; this framework already lives in CPython, so the executioner runs the code with ``exec`` in
a named context dictionary, converts INDArrays to numpy on the way in and numpy arrays / torch tensors back to INDArrays on the way
out, and keeps the GIL / context API so callers written against the reference keep working."""
from __future__ import annotations

import threading

import numpy as np
import torch

from ..nd.ndarray import INDArray


class PythonType:
    def __init__(self, name, py, to_py, from_py):
        self.name, self.py, self._to, self._from = name, py, to_py, from_py

    def getName(self): return self.name
    def toPython(self, v): return self._to(v)
    def toJava(self, v): return self._from(v)
    adapt = toJava


def _nd_to_py(v):
    return v.numpy() if isinstance(v, INDArray) else (v.detach().cpu().numpy() if isinstance(v, torch.Tensor) else np.asarray(v))


def _py_to_nd(v):
    if isinstance(v, INDArray):
        return v
    if isinstance(v, torch.Tensor):
        return INDArray(v)
    return INDArray(torch.as_tensor(np.asarray(v)))


class PythonTypes:
    STR = PythonType("str", str, str, str)
    INT = PythonType("int", int, int, int)
    FLOAT = PythonType("float", float, float, float)
    BOOL = PythonType("bool", bool, bool, bool)
    LIST = PythonType("list", list, list, list)
    DICT = PythonType("dict", dict, dict, dict)
    BYTES = PythonType("bytes", bytes, bytes, bytes)
    NDARRAY = PythonType("numpy.ndarray", np.ndarray, _nd_to_py, _py_to_nd)

    @staticmethod
    def get(name):
        for t in (PythonTypes.STR, PythonTypes.INT, PythonTypes.FLOAT, PythonTypes.BOOL, PythonTypes.LIST, PythonTypes.DICT,
                  PythonTypes.BYTES, PythonTypes.NDARRAY):
            if t.name == name:
                return t
        raise ValueError(f"unknown python type {name}")

    @staticmethod
    def getPythonTypeForJavaObject(v):
        if isinstance(v, (INDArray, np.ndarray, torch.Tensor)):
            return PythonTypes.NDARRAY
        for t in (PythonTypes.BOOL, PythonTypes.INT, PythonTypes.FLOAT, PythonTypes.STR, PythonTypes.BYTES, PythonTypes.LIST, PythonTypes.DICT):
            if isinstance(v, t.py):
                return t
        raise ValueError(f"no python type for {type(v)}")


class PythonVariable:
    def __init__(self, name, type_=None, value=None):
        self.name, self.value = name, value
        self.type = type_ or (PythonTypes.getPythonTypeForJavaObject(value) if value is not None else None)

    def getName(self): return self.name
    def getType(self): return self.type
    def getValue(self): return self.value
    def setValue(self, v): self.value = v


class PythonVariables(list):
    def add(self, name, type_=None, value=None):
        self.append(PythonVariable(name, type_, value))
        return self

    def get(self, name):
        return next(v for v in self if v.name == name)


class PythonGIL:
    """Reentrant lock standing in for GIL acquisition (``try (PythonGIL gil = PythonGIL.lock())``)."""
    _lock = threading.RLock()

    @staticmethod
    def lock():
        return PythonGIL()

    def __enter__(self):
        PythonGIL._lock.acquire()
        return self

    def __exit__(self, *a):
        PythonGIL._lock.release()

    close = __exit__

    @staticmethod
    def locked():
        return True


class PythonContextManager:
    """Named global dictionaries so independent snippets do not see each other's variables."""
    _contexts = {"main": {}}
    _current = "main"

    @staticmethod
    def setContext(name):
        PythonContextManager._contexts.setdefault(name, {})
        PythonContextManager._current = name

    @staticmethod
    def getCurrentContext(): return PythonContextManager._current

    @staticmethod
    def deleteContext(name):
        if name == "main":
            raise ValueError("cannot delete the main context")
        PythonContextManager._contexts.pop(name, None)
        if PythonContextManager._current == name:
            PythonContextManager._current = "main"

    @staticmethod
    def deleteNonMainContexts():
        for n in [n for n in PythonContextManager._contexts if n != "main"]:
            PythonContextManager.deleteContext(n)

    @staticmethod
    def reset():
        PythonContextManager._contexts[PythonContextManager._current] = {}

    @staticmethod
    def globals_():
        return PythonContextManager._contexts[PythonContextManager._current]


class PythonExecutioner:
    @staticmethod
    def setVariable(name, value):
        PythonContextManager.globals_()[name] = value

    @staticmethod
    def getVariable(name, type_=None):
        v = PythonContextManager.globals_()[name]
        return type_.toJava(v) if type_ is not None else v

    @staticmethod
    def exec(code, inputs=None, outputs=None):
        """Run ``code`` with ``inputs`` bound by name; afterwards every variable of ``outputs`` is read back and converted."""
        with PythonGIL.lock():
            g = PythonContextManager.globals_()
            for v in inputs or []:
                g[v.name] = v.type.toPython(v.value) if v.type is not None else v.value
            exec(compile(code, "<python4j>", "exec"), g)          # noqa: S102 (this module's purpose)
            for v in outputs or []:
                if v.name not in g:
                    raise KeyError(f"python code did not define output variable '{v.name}'")
                t = v.type or PythonTypes.getPythonTypeForJavaObject(g[v.name])
                v.type = t
                v.value = t.toJava(g[v.name])
        return outputs

    @staticmethod
    def execAndReturnAllVariables(code, inputs=None):
        with PythonGIL.lock():
            g = PythonContextManager.globals_()
            before = set(g)
            PythonExecutioner.exec(code, inputs, None)
            out = PythonVariables()
            for k in g:
                if k not in before and not k.startswith("__"):
                    try:
                        out.add(k, None, PythonTypes.getPythonTypeForJavaObject(g[k]).toJava(g[k]))
                    except ValueError:
                        pass
            return out


class PythonJob:
    """A snippet with ``setup()`` run once and ``run(**inputs)`` per call (``PythonJob.builder().code(...).setupRunMode(true)``)."""

    def __init__(self, name="job", code="", setupRunMode=False, context=None):
        self.name, self.code, self.setupRunMode = name, code, setupRunMode
        self.context = context or f"job_{name}"
        self._ready = False

    def setup(self):
        PythonContextManager.setContext(self.context)
        PythonExecutioner.exec(self.code)
        if self.setupRunMode:
            PythonExecutioner.exec("setup()")
        self._ready = True
        PythonContextManager.setContext("main")

    def exec(self, inputs=None, outputs=None):
        if not self._ready:
            self.setup()
        PythonContextManager.setContext(self.context)
        try:
            if self.setupRunMode:
                g = PythonContextManager.globals_()
                args = {v.name: (v.type.toPython(v.value) if v.type else v.value) for v in inputs or []}
                res = g["run"](**args) or {}
                for v in outputs or []:
                    t = v.type or PythonTypes.getPythonTypeForJavaObject(res[v.name])
                    v.type, v.value = t, t.toJava(res[v.name])
            else:
                PythonExecutioner.exec(self.code, inputs, outputs)
        finally:
            PythonContextManager.setContext("main")
        return outputs
