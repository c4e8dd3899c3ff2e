"""``TrainingClient``: ordered, dependency-chained asynchronous training operations.

Every call validates and packs its batch locally, registers an operation request
with the run (earlier pending requests become explicit dependencies), uploads
the input with back-pressure, and returns a future whose ``result()`` is a
``TrainingResult``. Staging is bounded by ``max_staging_bytes`` and
``max_pending_requests``. Reference: packages/client/src/shadowspill_client/training.py:117-1043.
"""
from __future__ import annotations

import concurrent.futures as cf
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Any

from .packing import BatchError, BatchValidator, pack_batch
from .protocol import OperationRequest, OperationResult, decode_array, encode_microbatches
from .text import Datum
from .transport import HTTPTransport, TransportError


@dataclass
class TrainingResult:
    loss: float | None
    metrics: dict[str, float]
    completed_updates: int
    execution_seconds: float
    request_id: str
    outputs: dict[str, Any] = field(default_factory=dict)


class OperationFuture(cf.Future):
    """The pending result of one submitted request. ``request_id`` is fixed at submission, so a
    caller that loses its connection can look the request up again instead of submitting it twice;
    ``accepted()`` resolves once the service has registered the request and holds its input, after
    which the request goes on even if this client goes away (it fails with the request's own error
    if that happens first). Reference: packages/client/src/shadowspill_client/results.py:154."""

    def __init__(self, request_id: str, operation: str):
        super().__init__()
        self.request_id, self.operation = request_id, operation
        self._acceptance: cf.Future = cf.Future()

    def accepted(self) -> cf.Future:
        return self._acceptance

    def _accept(self, state: dict) -> None:
        if not self._acceptance.done():
            self._acceptance.set_result(state)

    def _finish(self, source: cf.Future) -> None:
        exc = source.exception()
        if exc is not None:
            if not self._acceptance.done():
                self._acceptance.set_exception(exc)
            self.set_exception(exc)
        else:
            self._accept({"request_id": self.request_id, "state": "completed"})
            self.set_result(source.result())


class OperationFailed(RuntimeError):
    def __init__(self, result: OperationResult):
        self.result = result
        super().__init__(f"{result.state}: {result.error} (effect: {result.effect})")


class TrainingClient:
    def __init__(self, transport: HTTPTransport, session: str, run: str, info: dict[str, Any],
                 max_staging_bytes: int = 1 << 30, max_pending_requests: int = 8):
        self.transport, self.session, self.run = transport, session, run
        self.route = f"/v1/runs/{session}/{run}"
        self.info = info
        geo = info["geometry"]
        self.microbatch_tokens, self.microbatches = geo["microbatch_tokens"], geo["microbatches"]
        self.slots, self.vocab, self.workers = geo["slots"], geo["vocab_size"], geo["workers"]
        self.packing = geo.get("packing", "best_fit")
        plan = info.get("plan_summary") or {}
        estimates = {"step": plan.get("duration_seconds")} if plan.get("duration_seconds") else {}
        for op, summary in (info.get("operation_plans") or {}).items():
            if summary.get("duration_seconds"):
                estimates[op] = summary["duration_seconds"]
        self.validator = BatchValidator(self.vocab, self.microbatch_tokens,
                                        self.microbatches * self.workers, self.slots,
                                        tuple(geo.get("extra_fields", ())), estimates, self.packing)
        self.writer_id = uuid.uuid4().hex
        self.transport.request("POST", f"{self.route}/writers/{self.writer_id}", {})
        self.pool = cf.ThreadPoolExecutor(max_workers=max(2, max_pending_requests))
        # transfers wait on operations: they get threads of their own so they can never starve them
        self._downloads = cf.ThreadPoolExecutor(max_workers=2)
        self.max_staging_bytes, self.max_pending = max_staging_bytes, max_pending_requests
        self._lock = threading.Condition()
        self._pending: dict[str, cf.Future] = {}
        self._staged = 0
        self._closed = False
        self._local_metrics: list[dict[str, Any]] = []

    # ------------------------------------------------------------------ batches
    def validate_batch(self, datums: list[Datum], operation: str = "step", groups=None):
        """Checks a batch on this machine, before anything is uploaded: field shapes and values,
        the run's token and sequence capacities, and whether the batch packs into the run's
        microbatches. Returns a ``BatchValidation`` (totals, the packing strategy that worked,
        the plan's simulated time for ``operation``); raises ``BatchError`` otherwise."""
        return self.validator.validate(datums, operation, groups)

    def _pack(self, datums: list[Datum], placement: list | None = None, groups=None) -> bytes:
        self.validator.validate(datums, check_packing=False)
        mbs = pack_batch(datums, microbatch_tokens=self.microbatch_tokens,
                         microbatches=self.microbatches * self.workers, slots=self.slots,
                         policy=self.packing, placement=placement, groups=groups)
        return encode_microbatches(mbs)

    # ------------------------------------------------------------------ submission
    def _submit(self, operation: str, payload: bytes | None = None, **arguments) -> cf.Future:
        if self._closed:
            raise RuntimeError("training client is closed")
        size = len(payload) if payload else 0
        with self._lock:
            while (len(self._pending) >= self.max_pending or
                   (self._staged and self._staged + size > self.max_staging_bytes)):
                self._lock.wait(0.05)
            deps = list(self._pending)
            req = OperationRequest(operation, dependencies=deps, arguments=arguments,
                                   has_input=payload is not None, writer_id=self.writer_id)
            self._staged += size
            fut = OperationFuture(req.request_id, operation)
            self.pool.submit(self._drive, req, payload, fut).add_done_callback(fut._finish)
            self._pending[req.request_id] = fut

        def done(_f, rid=req.request_id, n=size):
            with self._lock:
                self._pending.pop(rid, None)
                self._staged -= n
                self._lock.notify_all()
        fut.add_done_callback(done)
        return fut

    def _drive(self, req: OperationRequest, payload: bytes | None, watcher: OperationFuture | None = None
               ) -> TrainingResult:
        body = {"operation": req.operation, "request_id": req.request_id,
                "dependencies": req.dependencies, "arguments": req.arguments,
                "has_input": req.has_input, "writer_id": req.writer_id, "digest": req.digest()}
        self.transport.request("POST", f"{self.route}/requests", body)
        if payload is not None:
            delay = 0.05
            while True:
                try:
                    self.transport.request("PUT", f"{self.route}/requests/{req.request_id}/input", payload)
                    break
                except TransportError as exc:
                    if exc.status != 429:      # back-pressure: the server asks to retry later
                        raise
                    time.sleep(delay)
                    delay = min(1.0, delay * 2)
        if watcher is not None:
            watcher._accept({"request_id": req.request_id, "state": "accepted", "operation": req.operation,
                             "dependencies": list(req.dependencies)})
        while True:
            _, data = self.transport.request("GET", f"{self.route}/requests/{req.request_id}",
                                             query={"wait": "completed", "timeout": 30})
            res = OperationResult(**data)
            if res.done:
                break
        if res.state != "completed":
            raise OperationFailed(res)
        return TrainingResult(res.loss, res.metrics, res.completed_updates, res.execution_seconds,
                              res.request_id, res.outputs)

    # ------------------------------------------------------------------ operations
    def step(self, datums: list[Datum], *, lr: float | None = None, grad_scale: float = 1.0,
             groups=None) -> cf.Future:
        """Forward, backward and one optimizer update on one global batch. ``grad_scale``
        multiplies the gradients inside the update (loss-scale compensation, caller-side clipping).
        ``groups``: lists of datum indices that must share a microbatch."""
        return self._submit("step", self._pack(datums, groups=groups), lr=lr, grad_scale=grad_scale)

    def forward_backward(self, datums: list[Datum], *, groups=None) -> cf.Future:
        """Accumulates gradients; the first contribution after an update writes them fresh."""
        return self._submit("forward_backward", self._pack(datums, groups=groups))

    def optim_step(self, *, grad_scale: float = 1.0, lr: float | None = None) -> cf.Future:
        return self._submit("optim_step", None, grad_scale=grad_scale, lr=lr)

    def forward(self, datums: list[Datum], mode: str = "evaluation") -> cf.Future:
        """Evaluates the batch without touching state. The result's ``loss`` is the objective;
        ``outputs["per_datum"]`` holds one float32 array per datum, row for row: for language
        models ``[n, 1]`` with the log-probability of each position's target (0 where there is
        none), for the regression family the ``[1, outputs]`` prediction."""
        placement: list = []
        inner = self._submit("forward", self._pack(datums, placement), mode=mode)

        outer: cf.Future = cf.Future()

        def unpack(done: cf.Future) -> None:      # runs on the thread that completed `inner`
            try:
                res = done.result()
                per_mb = [decode_array(a) for a in res.outputs.get("per_microbatch", [])]
                if per_mb:
                    res.outputs = {k: v for k, v in res.outputs.items() if k != "per_microbatch"}
                    res.outputs["per_datum"] = [per_mb[m][lo:lo + n] for m, lo, n in placement]
                outer.set_result(res)
            except BaseException as exc:  # noqa: BLE001
                outer.set_exception(exc)
        inner.add_done_callback(unpack)
        return outer

    def discard_gradients(self) -> cf.Future:
        return self._submit("discard", None)

    def save_checkpoint(self, name: str, metadata: dict | None = None) -> cf.Future:
        return self._submit("save", None, name=name, metadata=metadata or {})

    def load_checkpoint(self, checkpoint_id: str) -> cf.Future:
        return self._submit("restore", None, name=checkpoint_id)

    def export_weights(self, name: str) -> cf.Future:
        return self._submit("export", None, name=name)

    def traced_step(self, datums: list[Datum], directory, *, lr: float | None = None) -> cf.Future:
        """One real training step with the runtime trace on (the run must have been created with
        ``Execution(runtime_trace=True)``). The future gives ``(TrainingResult, path)`` where
        ``path/rank<r>/`` holds ``runtime.html``, ``runtime.json`` and the per-task tables of
        each worker: measured against simulated times, transfers, idle attribution."""
        from pathlib import Path
        from .handles import ArtifactHandle, download_artifact
        inner = self._submit("step", self._pack(datums), lr=lr, runtime_trace=True)

        def work():
            import tarfile
            res = inner.result()
            h = res.outputs["trace"]
            root = Path(directory)
            root.mkdir(parents=True, exist_ok=True)
            archive = download_artifact(self.transport, ArtifactHandle(h["artifact"], int(h["size"]), h["sha256"]),
                                        root / "trace.tar")
            with tarfile.open(archive) as tar:
                tar.extractall(root, filter="data")
            archive.unlink()
            return res, root / "trace"
        return self._downloads.submit(work)

    def download_plan_report(self, directory) -> cf.Future:
        """Renders the run's plan report on the service (``index.html``, ``occupancy.html``,
        ``tasks.csv``, ``transfers.csv``, ``timeline.json/.svg``, ``summary.json``) and unpacks it
        under ``directory``; the future gives the report's path."""
        from pathlib import Path
        from .handles import ArtifactHandle, download_artifact
        inner = self._submit("plan_report", None)

        def work():
            import tarfile
            h = inner.result().outputs
            handle = ArtifactHandle(h["artifact"], int(h["size"]), h["sha256"])
            root = Path(directory)
            root.mkdir(parents=True, exist_ok=True)
            archive = download_artifact(self.transport, handle, root / "plan_report.tar")
            with tarfile.open(archive) as tar:
                tar.extractall(root, filter="data")
            archive.unlink()
            return root / "plan_report"
        return self._downloads.submit(work)

    def list_checkpoints(self) -> list[str]:
        return self.transport.request("GET", f"{self.route}/checkpoints")[1]["checkpoints"]

    def checkpoint_manifest(self, name: str) -> cf.Future:
        """What a saved checkpoint holds, without downloading it: per archive its size, metadata
        (update count, world size, dtype, generator states) and tensor names."""
        return self.pool.submit(lambda: self.transport.request("GET", f"{self.route}/checkpoints/{name}/manifest")[1])

    def download_checkpoint(self, name: str, directory, **kw) -> cf.Future:
        """Fetches a checkpoint saved by ``save_checkpoint`` (or ``export_weights``) from the
        service and unpacks it under ``directory``; the future gives the unpacked path. The
        transfer resumes if ``<name>.tar.part`` from an earlier attempt is still there."""
        from pathlib import Path
        from .handles import ArtifactHandle, download_artifact

        def work():
            import tarfile
            _, h = self.transport.request("POST", f"{self.route}/checkpoints/{name}/artifact", {})
            handle = ArtifactHandle(h["artifact"], int(h["size"]), h["sha256"])
            root = Path(directory)
            root.mkdir(parents=True, exist_ok=True)
            archive = download_artifact(self.transport, handle, root / f"{name}.tar", **kw)
            with tarfile.open(archive) as tar:
                tar.extractall(root, filter="data")
            archive.unlink()
            return root / name
        return self.pool.submit(work)

    # ------------------------------------------------------------------ observations
    def lookup_request(self, request_id: str, wait_seconds: float = 0.0):
        """The service's record of a request by the id fixed at submission (``OperationFuture.
        request_id``): what to do after a lost connection instead of submitting again. Returns the
        ``TrainingResult`` of a completed request, raises ``OperationFailed`` for a failed or rejected
        one, and returns ``None`` while it is still pending (``wait_seconds`` > 0 waits that long)."""
        query = {"wait": "completed", "timeout": min(float(wait_seconds), 120.0)} if wait_seconds > 0 else None
        _, data = self.transport.request("GET", f"{self.route}/requests/{request_id}", query=query)
        res = OperationResult(**data)
        if not res.done:
            return None
        if res.state != "completed":
            raise OperationFailed(res)
        return TrainingResult(res.loss, res.metrics, res.completed_updates, res.execution_seconds,
                              res.request_id, res.outputs)

    @property
    def metrics(self):
        """Reads of this run's metric journal (``client.metrics.MetricQueries``)."""
        from .metrics import MetricQueries
        if getattr(self, "_metrics", None) is None:
            self._metrics = MetricQueries(self.transport, self.session, self.run, self._downloads)
        return self._metrics

    def log_metrics(self, step: int, **values: float) -> None:
        self.transport.request("POST", f"{self.route}/metrics", {"step": step, "values": values})

    def report(self, directory: str | None = None) -> dict:
        _, data = self.transport.request("POST", f"{self.route}/report", {"directory": directory})
        return data

    def close(self) -> None:
        if self._closed:
            return
        try:
            self._submit("close", None).result()
        finally:
            self._closed = True
            self.pool.shutdown(wait=False)
            self._downloads.shutdown(wait=False)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
