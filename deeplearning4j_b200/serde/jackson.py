"""Jackson-compatible JSON emission for DL4J configuration objects.

DL4J writes configurations with ``SORT_PROPERTIES_ALPHABETICALLY`` + ``INDENT_OUTPUT``
(``deeplearning4j-nn/.../nn/conf/serde/JsonMapperUtil.java:28-33``) and polymorphic ``@class``
type ids (``nn/conf/layers/Layer.java:51``).  This module reproduces Jackson's
``DefaultPrettyPrinter`` spacing (`` : `` separators, two-space indent, ``[ a, b ]`` arrays,
``{ }`` / ``[ ]`` for empties) and Java's ``Double.toString`` number formatting so that the
``configuration.json`` entry of a checkpoint is byte-stable across save/load.
"""
from __future__ import annotations

import json
import math
from typing import Any


class JavaFloat(float):
    """A value Java would print with ``Float.toString`` (kept distinct from double)."""


def java_double(v: float) -> str:
    """``Double.toString`` semantics: shortest repr, ``E`` notation outside [1e-3, 1e7)."""
    if math.isnan(v):
        return '"NaN"'
    if math.isinf(v):
        return '"Infinity"' if v > 0 else '"-Infinity"'
    if v == 0:
        return "-0.0" if math.copysign(1.0, v) < 0 else "0.0"
    from decimal import Decimal
    sign, digits, exp = Decimal(repr(float(v))).as_tuple()
    digits = list(digits)
    while len(digits) > 1 and digits[-1] == 0:
        digits.pop()
        exp += 1
    n = len(digits)
    sci = exp + n - 1          # exponent of the leading digit
    neg = "-" if sign else ""
    ds = "".join(map(str, digits))
    if -3 <= sci < 7:
        if sci >= 0:
            ip = ds[:sci + 1].ljust(sci + 1, "0")
            fp = ds[sci + 1:] or "0"
        else:
            ip = "0"
            fp = "0" * (-sci - 1) + ds
        return f"{neg}{ip}.{fp}"
    return f"{neg}{ds[0]}.{ds[1:] or '0'}E{sci}"


def _is_scalar(v):
    return v is None or isinstance(v, (bool, int, float, str))


def _scalar(v) -> str:
    if v is None:
        return "null"
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, int):
        return str(v)
    if isinstance(v, float):
        return java_double(v)
    return json.dumps(v, ensure_ascii=False)


def dumps(obj: Any, sort_keys: bool = True) -> str:
    """Serialise ``obj`` (dict / list / scalar tree) like Jackson's indented writer."""
    out: list[str] = []

    def emit(v, level: int):
        if isinstance(v, dict):
            if not v:
                out.append("{ }")
                return
            keys = list(v.keys())
            if sort_keys:
                # Jackson puts the type id first, then alphabetical properties
                keys = sorted(k for k in keys if k != "@class")
                if "@class" in v:
                    keys.insert(0, "@class")
            out.append("{\n")
            for i, k in enumerate(keys):
                out.append("  " * (level + 1) + json.dumps(k) + " : ")
                emit(v[k], level + 1)
                out.append(",\n" if i + 1 < len(keys) else "\n")
            out.append("  " * level + "}")
        elif isinstance(v, (list, tuple)):
            if not v:
                out.append("[ ]")
                return
            out.append("[ ")
            for i, e in enumerate(v):
                emit(e, level)
                if i + 1 < len(v):
                    out.append(", ")
            out.append(" ]")
        else:
            out.append(_scalar(v))

    emit(obj, 0)
    return "".join(out)


def loads(s: str):
    def _const(c):
        return {"NaN": float("nan"), "Infinity": float("inf"), "-Infinity": float("-inf")}[c]
    return json.loads(s, parse_constant=_const)
