"""Frozen, validated, JSON-portable settings records (no third-party imports).

Reference: packages/client/src/shadowspill_client/_records.py and config/*.py.
"""
from __future__ import annotations

import dataclasses
import json
from typing import Any


class ConfigError(ValueError):
    pass


def record(cls):
    """Frozen dataclass with ``to_json`` / ``from_json`` and ``validate`` on construction."""
    orig_post = cls.__dict__.get("__post_init__")

    def __post_init__(self):
        if orig_post:
            orig_post(self)
        v = getattr(self, "validate", None)
        if v:
            v()

    # the generated __init__ only calls a __post_init__ that exists when the class is decorated
    cls.__post_init__ = __post_init__
    cls = dataclasses.dataclass(frozen=True)(cls)

    def to_json(self) -> dict[str, Any]:
        out = {}
        for f in dataclasses.fields(self):
            val = getattr(self, f.name)
            if hasattr(val, "to_json"):
                val = val.to_json()
            elif isinstance(val, tuple):
                val = [x.to_json() if hasattr(x, "to_json") else x for x in val]
            out[f.name] = val
        out["_record"] = cls.__name__
        return out

    @classmethod
    def from_json(klass, d: dict[str, Any]):
        kw = {}
        hints = {f.name: f for f in dataclasses.fields(klass)}
        for k, v in d.items():
            if k == "_record" or k not in hints:
                continue
            if isinstance(v, dict) and "_record" in v:
                v = REGISTRY[v["_record"]].from_json(v)
            elif isinstance(v, list):
                v = tuple(REGISTRY[x["_record"]].from_json(x) if isinstance(x, dict) and "_record" in x
                          else x for x in v)
            kw[k] = v
        return klass(**kw)

    cls.to_json = to_json
    cls.from_json = from_json
    cls.digest = lambda self: __import__("hashlib").sha256(
        json.dumps(self.to_json(), sort_keys=True).encode()).hexdigest()
    REGISTRY[cls.__name__] = cls
    return cls


REGISTRY: dict[str, Any] = {}


def require(cond: bool, msg: str) -> None:
    if not cond:
        raise ConfigError(msg)
