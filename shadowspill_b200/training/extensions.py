"""Extension packages: components that a service loads at start.

A service imports every module named in ``SHADOWSPILL_EXTENSIONS`` (comma separated, or the
``extensions`` argument of ``Server``) and calls its ``register(registry)``. What the module adds
is listed with the module as its distribution, the module's ``__version__`` and a digest of the
component's source, so a run's provenance says which code defined its model or policy. An id that
exists already is refused: an extension adds, it never replaces. A module that cannot be imported,
has no ``register`` or raises inside it stops the service start with the module named.

Reference: the reference's extension packages (examples/extensions/custom_training, loaded through
its component registry: packages/engine/src/shadowspill/training/components/registry.py).
"""
from __future__ import annotations

import dataclasses
import importlib
import os


class ExtensionError(RuntimeError):
    pass


def requested(names=None) -> list[str]:
    if names is None:
        names = os.environ.get("SHADOWSPILL_EXTENSIONS", "").split(",")
    return [n.strip() for n in names if n and n.strip()]


def load_extensions(registry, names=None) -> dict[str, list[str]]:
    """Returns ``{module: [component ids it added]}``."""
    added: dict[str, list[str]] = {}
    for name in requested(names):
        before = set(registry._items)
        try:
            module = importlib.import_module(name)
        except Exception as exc:  # noqa: BLE001
            raise ExtensionError(f"extension {name!r} cannot be imported: {type(exc).__name__}: {exc}") from exc
        register = getattr(module, "register", None)
        if not callable(register):
            raise ExtensionError(f"extension {name!r} has no register(registry) function")
        try:
            register(registry)
        except Exception as exc:  # noqa: BLE001
            raise ExtensionError(f"extension {name!r} failed while registering: {type(exc).__name__}: {exc}") from exc
        new = [key for key in registry._items if key not in before]
        version = str(getattr(module, "__version__", "0"))
        for key in new:
            comp = registry._items[key]
            comp.source = dataclasses.replace(comp.source, distribution=name, version=version)
        added[name] = [f"{kind}:{cid}" for kind, cid in new]
    return added
