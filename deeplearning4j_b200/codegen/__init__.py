"""Op-namespace code generation (``codegen/op-codegen``: op definitions -> the ``NDMath`` / ``SDMath`` ... namespace classes).

The reference describes every op in a Kotlin DSL and generates Java namespaces from it.  Here the op registry is the single source:
``describe()`` turns a registered op into a descriptor (name, group, inputs, keyword arguments with defaults, output count),
``generate_namespace_source(group)`` renders a Python namespace class with one documented method per op of that group (ND4J style,
eager) and ``generate_docs()`` renders the Markdown op list; ``write_all(dir)`` writes one file per group."""
from __future__ import annotations

import inspect
import keyword
import os

from ..ops import registry

GROUP_CLASS = {"elementwise": "NDMath", "reduce": "NDBase", "shape": "NDBase", "nn": "NDNN", "conv": "NDCNN", "rnn": "NDRNN", "loss": "NDLoss",
               "linalg": "NDLinalg", "image": "NDImage", "random": "NDRandom", "misc": "NDBase", "updaters": "NDUpdaters"}


def describe(name):
    d = registry.get(name)
    sig = inspect.signature(d.fn)
    inputs, kwargs, varargs = [], [], None
    for p in sig.parameters.values():
        if p.kind == p.VAR_POSITIONAL:
            varargs = p.name
        elif p.kind == p.VAR_KEYWORD or p.name.startswith("_"):
            continue
        elif p.default is p.empty:
            inputs.append(p.name)
        else:
            kwargs.append((p.name, p.default))
    return {"name": name, "group": d.group, "n_out": d.n_out, "differentiable": getattr(d, "differentiable", True), "inputs": inputs,
            "varargs": varargs, "args": kwargs}


def _ident(n):
    n = "".join(c if c.isalnum() else "_" for c in n)
    if n[0].isdigit():
        n = "_" + n
    return n + "_" if keyword.iskeyword(n) else n


def _plain(v):
    """Default values that can be written back as source text."""
    if type(v) in (int, float, str, bool, type(None)):
        return v == v and v not in (float("inf"), float("-inf"))
    return type(v) in (tuple, list) and all(_plain(e) for e in v)


def generate_namespace_source(group, class_name=None):
    cls = class_name or GROUP_CLASS.get(group, "ND" + group.capitalize())
    lines = [f'"""Generated from the op registry: ops of group \'{group}\'."""', "from deeplearning4j_b200.ops import registry", "", "",
             f"class {cls}:"]
    names = [n for n in registry.names() if registry.get(n).group == group]
    if not names:
        lines.append("    pass")
    for n in sorted(names):
        d = describe(n)
        params = [_ident(i) for i in d["inputs"]]
        if d["varargs"]:
            params.append("*" + _ident(d["varargs"]))
        kw = [f"{_ident(k)}={v!r}" if _plain(v) else f"{_ident(k)}=None" for k, v in d["args"]]
        call_in = ", ".join([_ident(i) for i in d["inputs"]] + (["*" + _ident(d["varargs"])] if d["varargs"] else []))
        call_kw = ", ".join(f"{k}={_ident(k)}" for k, _ in d["args"])
        lines += [f"    @staticmethod", f"    def {_ident(n)}({', '.join(params + kw)}):",
                  f'        """``{n}``: {len(d["inputs"])} input(s){" + varargs" if d["varargs"] else ""}, {d["n_out"] if d["n_out"] > 0 else "variable"} output(s)."""',
                  f"        return registry.execute({n!r}, [{call_in}]{', ' + call_kw if call_kw else ''})", ""]
    return "\n".join(lines) + "\n"


def generate_docs():
    out = ["# Operations", ""]
    by = {}
    for n in registry.names():
        by.setdefault(registry.get(n).group, []).append(n)
    for g in sorted(by):
        out += [f"## {g} ({len(by[g])})", ""]
        for n in sorted(by[g]):
            d = describe(n)
            args = ", ".join(d["inputs"] + ([f"*{d['varargs']}"] if d["varargs"] else []) + [f"{k}={v!r}" for k, v in d["args"]])
            out.append(f"* `{n}({args})`")
        out.append("")
    return "\n".join(out)


def write_all(directory):
    os.makedirs(directory, exist_ok=True)
    written = []
    for g in sorted({registry.get(n).group for n in registry.names()}):
        if not g or "." in g:
            continue
        p = os.path.join(directory, f"{GROUP_CLASS.get(g, 'ND' + g.capitalize()).lower()}_{g}.py")
        with open(p, "w") as f:
            f.write(generate_namespace_source(g, GROUP_CLASS.get(g, "ND" + g.capitalize()) + g.capitalize()))
        written.append(p)
    with open(os.path.join(directory, "ops.md"), "w") as f:
        f.write(generate_docs())
    return written
