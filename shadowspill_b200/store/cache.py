"""A small content-addressed store on disk.

An entry is addressed by the SHA-256 of its *key record* (a JSON value naming everything the
result depends on: device, kernel library digest, profile key, ...). Values are JSON; writes go
to a temporary file and are renamed into place, so concurrent workers can share one store.
``StoreMode`` says what a session may do with it: ``off``, ``read`` (never write), ``read_write``
or ``refresh`` (ignore what is there, write new results).

Used for task profiles: timing a task depends only on the device, the kernel library and the
task's profile key, so a second run with the same model and geometry skips the profiling phase.
Reference: packages/engine/src/shadowspill/store/ (content-addressed cache + ``StoreMode``).
"""
from __future__ import annotations

import hashlib
import json
import os
import tempfile
from enum import Enum
from pathlib import Path
from typing import Any


class StoreMode(str, Enum):
    OFF = "off"
    READ = "read"
    READ_WRITE = "read_write"
    REFRESH = "refresh"


def _address(kind: str, key: Any) -> str:
    blob = json.dumps({"kind": kind, "key": key}, sort_keys=True, default=str).encode()
    return hashlib.sha256(blob).hexdigest()


class ContentStore:
    def __init__(self, root: str | os.PathLike, mode: StoreMode | str = StoreMode.READ_WRITE):
        self.root = Path(root)
        self.mode = StoreMode(mode)
        self.hits = self.misses = self.writes = 0

    def _path(self, address: str) -> Path:
        return self.root / address[:2] / f"{address}.json"

    def get(self, kind: str, key: Any) -> Any | None:
        if self.mode in (StoreMode.OFF, StoreMode.REFRESH):
            return None
        p = self._path(_address(kind, key))
        try:
            rec = json.loads(p.read_text())
        except (OSError, ValueError):
            self.misses += 1
            return None
        if rec.get("kind") != kind or rec.get("key") != json.loads(json.dumps(key, default=str)):
            self.misses += 1          # an address collision or a damaged entry: treat as absent
            return None
        self.hits += 1
        return rec["value"]

    def put(self, kind: str, key: Any, value: Any) -> bool:
        if self.mode in (StoreMode.OFF, StoreMode.READ):
            return False
        p = self._path(_address(kind, key))
        p.parent.mkdir(parents=True, exist_ok=True)
        fd, tmp = tempfile.mkstemp(prefix=p.name + ".", suffix=".tmp", dir=p.parent)
        try:
            with os.fdopen(fd, "w") as f:
                json.dump({"kind": kind, "key": json.loads(json.dumps(key, default=str)), "value": value}, f)
                f.flush()
                os.fsync(f.fileno())
            os.replace(tmp, p)
        except BaseException:
            try:
                os.unlink(tmp)
            except FileNotFoundError:
                pass
            raise
        self.writes += 1
        return True


def kernel_library_digest() -> str:
    """Digest of the built kernel library: a profile is valid only for the kernels it timed."""
    from ..ops import _lib
    path = Path(_lib.__file__).with_name("libss_kernels.so")
    h = hashlib.sha256()
    try:
        with open(path, "rb") as f:
            for block in iter(lambda: f.read(1 << 20), b""):
                h.update(block)
    except OSError:
        return "unbuilt"
    return h.hexdigest()[:32]
