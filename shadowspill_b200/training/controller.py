"""Run controller: accepts ordered operation requests and dispatches them one at a
time to the worker group, with the accumulation state machine, writer fencing
and durable receipts.

State rules (reference: packages/engine/src/shadowspill/training/session/
{controller.py:39,134-257, state.py:37-63, writers.py} and
docs/python/advanced/service-client.md:304-358):
  * one command in flight; state changes only at confirmed completion;
  * ``step``, ``save``, ``restore`` and ``close`` need closed accumulation;
    ``forward_backward`` opens/extends it, ``optim_step`` applies it once,
    ``discard`` drops it;
  * a worker failure with unknown effect invalidates the state: only ``close``
    is accepted afterwards, and an uncertain update is never replayed;
  * requests are idempotent by digest: re-registering an identical request
    returns its status, a different body under the same id is rejected;
  * a newer writer fences every older one.
"""
from __future__ import annotations

import threading
import time
from dataclasses import asdict, dataclass, field
from typing import Any, Callable

from ..client.protocol import OperationResult


class Rejected(ValueError):
    pass


@dataclass
class Boundary:
    history_id: int = 0
    completed_updates: int = 0
    accumulation: int = 0
    valid: bool = True
    closed: bool = False


class OperationState:
    """Which commands the current boundary admits, and how completion moves it."""
    NEEDS_CLOSED_ACCUMULATION = ("step", "save", "restore", "export", "close")

    def __init__(self):
        self.b = Boundary()

    def admit(self, op: str) -> None:
        if self.b.closed:
            raise Rejected("the run is closed")
        if not self.b.valid and op != "close":
            raise Rejected("training state is invalid after a failed update; only close is accepted")
        if op in self.NEEDS_CLOSED_ACCUMULATION and self.b.accumulation and op != "close":
            raise Rejected(f"{op} needs closed accumulation: call optim_step or discard_gradients first")
        if op == "optim_step" and self.b.accumulation == 0:
            raise Rejected("optim_step without accumulated gradients")

    def complete(self, op: str) -> None:
        self.b.history_id += 1
        if op == "step":
            self.b.completed_updates += 1
        elif op == "forward_backward":
            self.b.accumulation += 1
        elif op == "optim_step":
            self.b.completed_updates += 1
            self.b.accumulation = 0
        elif op == "discard":
            self.b.accumulation = 0
        elif op == "close":
            self.b.closed = True

    def fail(self, effect: str) -> None:
        if effect == "unknown":
            self.b.valid = False


@dataclass
class _Entry:
    request: dict[str, Any]
    result: OperationResult
    payload: bytes | None = None
    event: threading.Event = field(default_factory=threading.Event)


class RunController:
    def __init__(self, execute: Callable[[dict[str, Any], bytes | None], dict[str, Any]],
                 journal=None, max_staging_bytes: int = 4 << 30, idle_timeout: float = 0.0):
        self.execute = execute
        self.journal = journal
        self.state = OperationState()
        self.max_staging = max_staging_bytes
        self.idle_timeout = idle_timeout
        self.entries: dict[str, _Entry] = {}
        self.order: list[str] = []
        self.writer: str | None = None
        self._staged = 0
        self._cv = threading.Condition()
        self._stop = False
        self._last_activity = time.monotonic()
        self.thread = threading.Thread(target=self._run, name="run-controller", daemon=True)
        self.thread.start()

    # ------------------------------------------------------------------ writers
    def attach_writer(self, writer_id: str) -> None:
        with self._cv:
            self.writer = writer_id          # fences every earlier writer
            if self.journal:
                self.journal.append("writer", {"writer_id": writer_id})

    # ------------------------------------------------------------------ intake
    def register(self, req: dict[str, Any]) -> OperationResult:
        with self._cv:
            rid = req["request_id"]
            if self.writer is not None and req.get("writer_id") != self.writer:
                raise Rejected("this writer has been fenced by a newer one")
            old = self.entries.get(rid)
            if old is not None:
                if old.request.get("digest") != req.get("digest"):
                    raise Rejected("request id reused with a different body")
                return old.result            # idempotent, never replays
            entry = _Entry(req, OperationResult(rid, "pending"))
            self.entries[rid] = entry
            self.order.append(rid)
            if self.journal:
                self.journal.append("accepted", {k: req[k] for k in
                                                 ("request_id", "operation", "dependencies", "digest")
                                                 if k in req})
            self._last_activity = time.monotonic()
            self._cv.notify_all()
            return entry.result

    def receive(self, request_id: str, payload: bytes) -> None:
        with self._cv:
            entry = self.entries.get(request_id)
            if entry is None:
                raise Rejected("unknown request")
            if self._staged + len(payload) > self.max_staging and self._staged > 0:
                raise BlockingIOError("staging area is full")      # -> HTTP 429 back-pressure
            entry.payload = payload
            self._staged += len(payload)
            self._cv.notify_all()

    def wait(self, request_id: str, timeout: float) -> OperationResult:
        entry = self.entries.get(request_id)
        if entry is None:
            raise Rejected("unknown request")
        entry.event.wait(timeout)
        return entry.result

    # ------------------------------------------------------------------ dispatch
    def _ready(self, entry: _Entry) -> bool:
        return not entry.request.get("has_input") or entry.payload is not None

    def _run(self) -> None:
        index = 0
        while True:
            with self._cv:
                while not self._stop and (index >= len(self.order) or
                                          not self._ready(self.entries[self.order[index]])):
                    self._cv.wait(0.1)
                    if (self.idle_timeout and index >= len(self.order) and
                            time.monotonic() - self._last_activity > self.idle_timeout):
                        self._stop = True
                if self._stop:
                    return
                entry = self.entries[self.order[index]]
            index += 1
            self._one(entry)
            if self.state.b.closed:
                return

    def _one(self, entry: _Entry) -> None:
        req, res = entry.request, entry.result
        op = req["operation"]
        try:
            for dep in req.get("dependencies", []):
                d = self.entries.get(dep)
                if d is not None and d.result.state in ("failed", "rejected"):
                    raise Rejected(f"dependency {dep} did not complete")
            self.state.admit(op)
        except Rejected as exc:
            res.state, res.error = "rejected", str(exc)
            self._finish(entry)
            return
        res.state = "running"
        try:
            out = self.execute(req, entry.payload)
            self.state.complete(op)
            res.state, res.effect = "completed", "completed"
            res.loss = out.get("loss")
            res.metrics = out.get("metrics", {})
            res.outputs = out.get("outputs", {})
            res.execution_seconds = out.get("execution_seconds", 0.0)
        except Exception as exc:  # noqa: BLE001
            effect = getattr(exc, "effect", "unknown")
            self.state.fail(effect)
            res.state, res.effect, res.error = "failed", effect, str(exc)
        res.completed_updates = self.state.b.completed_updates
        self._finish(entry)

    def _finish(self, entry: _Entry) -> None:
        with self._cv:
            if entry.payload is not None:
                self._staged -= len(entry.payload)
                entry.payload = None
            if self.journal:
                r = entry.result
                self.journal.append("receipt", {"request_id": r.request_id, "state": r.state,
                                                "effect": r.effect, "loss": r.loss,
                                                "completed_updates": r.completed_updates,
                                                "operation": entry.request["operation"],
                                                "execution_seconds": r.execution_seconds,
                                                "error": r.error[:500]})
            self._last_activity = time.monotonic()
            entry.event.set()
            self._cv.notify_all()

    def boundary(self) -> dict[str, Any]:
        return asdict(self.state.b)

    def stop(self) -> None:
        with self._cv:
            self._stop = True
            self._cv.notify_all()
