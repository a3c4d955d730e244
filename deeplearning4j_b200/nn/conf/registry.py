"""``@class`` -> Python class registry for polymorphic JSON (layers, vertices, misc configs)."""
from __future__ import annotations

import importlib

_LAYER_MODULES = ("core", "conv", "recurrent", "attention", "special")
_CACHE = {}


def _scan():
    if _CACHE:
        return _CACHE
    from .base import Layer
    for m in _LAYER_MODULES:
        try:
            mod = importlib.import_module(f"deeplearning4j_b200.nn.layers.{m}")
        except ModuleNotFoundError as e:
            if f"layers.{m}" in str(e):
                continue
            raise
        for v in vars(mod).values():
            if isinstance(v, type) and issubclass(v, Layer) and getattr(v, "JAVA_CLASS", "").count(".") > 3:
                _CACHE.setdefault(v.JAVA_CLASS, v)
    return _CACHE


def layer_classes():
    return dict(_scan())


def layer_from_json(d):
    if d is None:
        return None
    reg = _scan()
    jc = d["@class"]
    cls = reg.get(jc)
    if cls is None:
        short = jc.rsplit(".", 1)[-1]
        for k, v in reg.items():
            if k.rsplit(".", 1)[-1] == short:
                cls = v
                break
    if cls is None:
        raise ValueError(f"unknown layer class {jc}")
    if "lambda" in d and "lambda_" in getattr(cls, "DEFAULTS", {}):
        d = dict(d)
        d["lambda_"] = d.pop("lambda")
    for key in ("layer", "underlying", "fwd", "bwd"):
        if isinstance(d.get(key), dict) and "@class" in d[key] and key in _wrapper_keys(cls):
            d = dict(d)
            d[key] = layer_from_json(d[key])
    obj = cls.from_json(d)
    return obj


def _wrapper_keys(cls):
    keys = set()
    for c in cls.__mro__:
        keys.update(k for k in getattr(c, "DEFAULTS", {}) if k in ("layer", "underlying", "fwd", "bwd"))
    return keys


def object_from_json(d):
    """Generic fallback for nested typed objects inside a layer config."""
    jc = d["@class"]
    if "ReconstructionDistribution" in jc or jc.endswith("variational.LossFunctionWrapper"):
        from ..layers.special import reconstruction_from_json
        return reconstruction_from_json(d)
    if ".layers." in jc:
        return layer_from_json(d)
    if ".preprocessor." in jc:
        from .preprocessors import preprocessor_from_json
        return preprocessor_from_json(d)
    if ".schedule." in jc:
        from ..updaters import schedule_from_json
        return schedule_from_json(d)
    if ".distribution." in jc:
        from ..weights import distribution_from_json
        return distribution_from_json(d)
    if ".lossfunctions." in jc:
        from ..losses import LossFunctions
        return LossFunctions.from_json(d)
    if ".activations." in jc:
        from ..activations import Activation
        return Activation.from_json(d)
    if "variational" in jc:
        from ..layers.special import reconstruction_from_json
        return reconstruction_from_json(d)
    return d
