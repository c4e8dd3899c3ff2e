"""Durable run journal: fsynced, hash-chained records, one file per record.

The journal is the authority for what a run has accepted and completed; metric
history and run listings are projections of it. Each record names the SHA-256 of
its predecessor, so truncation or tampering is detected on recovery.
Reference: packages/engine/src/shadowspill/server/records/journal.py:41.
"""
from __future__ import annotations

import hashlib
import json
import os
import threading
import time
from pathlib import Path
from typing import Any, Iterator


class JournalCorrupt(RuntimeError):
    pass


class Journal:
    def __init__(self, directory: str | Path):
        self.dir = Path(directory)
        self.dir.mkdir(parents=True, exist_ok=True)
        self._lock = threading.Lock()
        self.head = "0" * 64
        self.count = 0
        for rec in self._scan():
            self.head, self.count = rec["hash"], rec["seq"] + 1

    def _path(self, seq: int) -> Path:
        return self.dir / f"{seq:012d}.json"

    def _scan(self) -> Iterator[dict[str, Any]]:
        prev, seq = "0" * 64, 0
        while True:
            p = self._path(seq)
            if not p.exists():
                return
            try:
                rec = json.loads(p.read_text())
            except json.JSONDecodeError:
                raise JournalCorrupt(f"{p} is not valid JSON") from None
            body = {k: rec[k] for k in ("seq", "time", "kind", "data", "prev")}
            digest = hashlib.sha256(json.dumps(body, sort_keys=True).encode()).hexdigest()
            if rec["prev"] != prev or rec["hash"] != digest or rec["seq"] != seq:
                raise JournalCorrupt(f"{p} breaks the hash chain")
            yield rec
            prev, seq = rec["hash"], seq + 1

    def append(self, kind: str, data: dict[str, Any]) -> dict[str, Any]:
        with self._lock:
            body = {"seq": self.count, "time": time.time(), "kind": kind, "data": data,
                    "prev": self.head}
            rec = dict(body, hash=hashlib.sha256(json.dumps(body, sort_keys=True).encode()).hexdigest())
            tmp = self._path(self.count).with_suffix(".tmp")
            with open(tmp, "w") as f:
                f.write(json.dumps(rec))
                f.flush()
                os.fsync(f.fileno())
            os.replace(tmp, self._path(self.count))
            fd = os.open(self.dir, os.O_RDONLY)
            try:
                os.fsync(fd)
            finally:
                os.close(fd)
            self.head, self.count = rec["hash"], self.count + 1
            return rec

    def records(self, kind: str | None = None) -> list[dict[str, Any]]:
        return [r for r in self._scan() if kind is None or r["kind"] == kind]
