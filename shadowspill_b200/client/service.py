"""``ServiceClient``: connection to a training service.

Connecting is blocking; every later call returns a future run by a bounded
thread pool; nothing is retried automatically. Reference:
packages/client/src/shadowspill_client/service.py:49-611.
"""
from __future__ import annotations

import concurrent.futures as cf
import time
import uuid
from typing import Any

from .config import (BatchConfig, Execution, Memory, Model, Objective, Optimizer, Preparation,
                     Resources, training_setup)
from .training import TrainingClient
from .transport import HTTPTransport, TransportError


class ProgressDisplay:
    """Shows a run's preparation log while the run comes up: a stamped heading when the run's
    state changes, then the log lines that are new since the last poll (at most two polls a
    second). Display trouble never reaches the creation: the first error switches it off with one
    note. Reference: packages/client/src/shadowspill_client/_progress.py:19."""

    def __init__(self, target, run: str):
        import sys
        self.stream = sys.stdout if target is True else (target or None)
        self.run, self.seen, self.state, self.next_poll = run, 0, None, 0.0

    def update(self, transport, session: str, info: dict[str, Any], final: bool = False) -> None:
        if self.stream is None:
            return
        try:
            changed = info.get("state") != self.state
            if changed:
                self.state = info.get("state")
                stamp = time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())
                self.stream.write(f"\n{stamp}  Run {self.run[:12]} - {str(self.state).capitalize()}\n")
            if not final and not changed and time.monotonic() < self.next_poll:
                return
            self.next_poll = time.monotonic() + 0.5
            _, page = transport.request("GET", f"/v1/runs/{session}/{self.run}/progress", query={"after": self.seen})
            for line in page.get("lines", ()):
                self.stream.write(f"  {line}\n")
            self.seen = int(page.get("next", self.seen))
            self.stream.flush()
        except Exception as exc:  # noqa: BLE001
            stream, self.stream = self.stream, None
            try:
                stream.write(f"\n  ! live progress unavailable ({type(exc).__name__}); creation continues\n")
            except Exception:  # noqa: BLE001
                pass


class ServiceClient:
    def __init__(self, url: str | None = None, token: str = "", timeout: float = 600.0, max_workers: int = 8,
                 ssh=None, session: str | None = None):
        """``ssh`` (a ``client.transport.SSH``): reach the service through an OpenSSH forward that this
        client owns and closes with itself; ``url`` is then not given. ``session``: the id of an earlier
        client's session (``ServiceClient.session``), to reach its runs again from another process:
        ``get_training_client(run)`` then attaches as the run's writer and fences the earlier one."""
        self.tunnel = None
        if ssh is not None:
            if url:
                raise ValueError("give a url or ssh settings, not both")
            from .transport import SSHTunnel
            self.tunnel = SSHTunnel(ssh)
            url = self.tunnel.open()
        elif not url:
            raise ValueError("a service url (or ssh settings) is required")
        self.transport = HTTPTransport(url, token, timeout)
        try:
            _, self.info = self.transport.request("GET", "/v1/info")     # blocking connect
        except BaseException:
            if self.tunnel is not None:
                self.tunnel.close()
            raise
        self.pool = cf.ThreadPoolExecutor(max_workers=max_workers)
        if session is not None and (not isinstance(session, str) or not session.isalnum() or len(session) > 64):
            raise ValueError("a session id is a short alphanumeric string")
        self.session = session or uuid.uuid4().hex[:12]

    # ------------------------------------------------------------------ discovery
    def list_hardware(self) -> cf.Future:
        return self.pool.submit(lambda: self.transport.request("GET", "/v1/hardware")[1])

    def describe_training(self, **setup) -> cf.Future:
        """Resolves settings and previews workers and memory without reserving anything."""
        body = training_setup(**setup)
        return self.pool.submit(lambda: self.transport.request("POST", "/v1/training/describe", body)[1])

    # ------------------------------------------------------------------ runs
    def _create(self, body: dict[str, Any], wait: bool, timeout: float, progress=None) -> dict[str, Any]:
        _, info = self.transport.request("POST", f"/v1/runs/{self.session}", body)
        run = info["run"]
        deadline = time.monotonic() + timeout
        shown = ProgressDisplay(progress, run)
        while wait and info["state"] == "preparing":
            if time.monotonic() > deadline:
                raise TimeoutError("run did not become ready in time")
            time.sleep(0.2)
            _, info = self.transport.request("GET", f"/v1/runs/{self.session}/{run}")
            shown.update(self.transport, self.session, info)
        shown.update(self.transport, self.session, info, final=True)
        if info["state"] == "failed":
            raise RuntimeError(f"run creation failed: {info.get('error', '')}")
        return info

    def create_training_client(self, model: Model, optimizer: Optimizer = Optimizer(),
                               objective: Objective = Objective(), batch: BatchConfig = BatchConfig(),
                               memory: Memory = Memory(), execution: Execution = Execution(),
                               preparation: Preparation = Preparation(),
                               resources: Resources = Resources(), parallelism: dict | None = None,
                               operations: tuple = ("step",), plans: str | None = None,
                               checkpoint: str | None = None, timeout: float = 3600.0, progress=None) -> cf.Future:
        """``progress``: ``True`` (standard output) or a text stream: the run's preparation log
        (build, profile, calibrate, plan, worker start) is shown while the run comes up."""
        body = training_setup(model, optimizer, objective, batch, memory, execution, preparation,
                              resources, parallelism, operations)
        body["plans"], body["checkpoint"] = plans, checkpoint
        if hasattr(plans, "create_arguments"):            # a PlansHandle: a run of this session or an import
            body["plans"] = None
            body.update(plans.create_arguments())

        def work() -> TrainingClient:
            info = self._create(body, True, timeout, progress)
            return TrainingClient(self.transport, self.session, info["run"], info,
                                  execution.max_staging_bytes, execution.max_pending_requests)
        return self.pool.submit(work)

    def prepare_training(self, **setup) -> cf.Future:
        """Runs build/profile/plan only and stores the plans under the run."""
        body = training_setup(**setup)
        body["prepare_only"] = True
        return self.pool.submit(lambda: self._create(body, True, 3600.0))

    def plan_training(self, **setup) -> cf.Future:
        """Plans against modelled task costs without touching a GPU (simulation only)."""
        body = training_setup(**setup)
        body["prepare_only"], body["simulation_only"] = True, True
        return self.pool.submit(lambda: self._create(body, True, 3600.0))

    def plans_of(self, run: str):
        """The ``PlansHandle`` of a prepared (or running) run of this session."""
        from .handles import PlansHandle
        return PlansHandle(self, run)

    def import_plans(self, path, **kw) -> cf.Future:
        """Uploads a bundle that ``PlansHandle.export`` wrote; the future gives a ``PlansHandle``
        that new runs of this service accept as ``plans``."""
        from .handles import PlansHandle, upload_artifact
        return self.pool.submit(lambda: PlansHandle(self, None, upload_artifact(self.transport, path, **kw)))

    def wait_ready(self, run: str, timeout: float = 3600.0, progress=None) -> cf.Future:
        """Waits for a run of this session that is still preparing (a client that lost its
        connection during ``create_training_client`` or ``prepare_training`` picks the run up again
        by its id); the future gives the run's info, or raises if the preparation failed."""
        def work():
            deadline = time.monotonic() + timeout
            shown = ProgressDisplay(progress, run)
            while True:
                _, info = self.transport.request("GET", f"/v1/runs/{self.session}/{run}")
                shown.update(self.transport, self.session, info, final=info["state"] != "preparing")
                if info["state"] != "preparing":
                    break
                if time.monotonic() > deadline:
                    raise TimeoutError("run did not become ready in time")
                time.sleep(0.2)
            if info["state"] == "failed":
                raise RuntimeError(f"run creation failed: {info.get('error', '')}")
            return info
        return self.pool.submit(work)

    def get_training_client(self, run: str) -> cf.Future:
        """Attaches to a running run as its writer; any earlier writer is fenced."""
        def work():
            _, info = self.transport.request("GET", f"/v1/runs/{self.session}/{run}")
            return TrainingClient(self.transport, self.session, run, info)
        return self.pool.submit(work)

    # ------------------------------------------------------------------ observations
    def get_metrics(self, run: str, after: int = 0, limit: int = 1000) -> cf.Future:
        return self.pool.submit(lambda: self.transport.request(
            "GET", f"/v1/runs/{self.session}/{run}/metrics", query={"after": after, "limit": limit})[1])

    def get_plans(self, run: str, page: int = 0) -> cf.Future:
        return self.pool.submit(lambda: self.transport.request(
            "GET", f"/v1/runs/{self.session}/{run}/plans", query={"page": page})[1])

    def get_plan_report(self, run: str, directory: str | None = None) -> cf.Future:
        return self.pool.submit(lambda: self.transport.request(
            "POST", f"/v1/runs/{self.session}/{run}/plans/report", {"directory": directory})[1])

    def get_progress(self, run: str, after: int = 0) -> cf.Future:
        return self.pool.submit(lambda: self.transport.request(
            "GET", f"/v1/runs/{self.session}/{run}/progress", query={"after": after})[1])

    def list_components(self, kind: str | None = None) -> cf.Future:
        return self.pool.submit(lambda: self.transport.request(
            "GET", "/v1/components", query={"kind": kind} if kind else None)[1]["components"])

    def upload_artifact(self, path, **kw) -> cf.Future:
        """Resumable upload of a file (weights, a prepared bundle); returns an ``ArtifactHandle``."""
        from .handles import upload_artifact
        return self.pool.submit(lambda: upload_artifact(self.transport, path, **kw))

    def download_artifact(self, artifact, path, **kw) -> cf.Future:
        from .handles import download_artifact
        return self.pool.submit(lambda: download_artifact(self.transport, artifact, path, **kw))

    def delete_artifact(self, artifact) -> cf.Future:
        aid = getattr(artifact, "artifact", artifact)
        return self.pool.submit(lambda: self.transport.request("DELETE", f"/v1/artifacts/{aid}")[1])

    def get_nsys(self, run: str, rank: int = 0) -> cf.Future:
        return self.pool.submit(lambda: self.transport.request(
            "GET", f"/v1/runs/{self.session}/{run}/nsys", query={"rank": rank})[1])

    def close(self) -> None:
        self.pool.shutdown(wait=False)
        if self.tunnel is not None:
            self.tunnel.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
