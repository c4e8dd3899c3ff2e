"""Resumable artifact uploads and downloads.

An upload is begun with the file's size and SHA-256; the service answers with how many
bytes it already holds, chunks are appended from there, and sealing checks the digest. A
chunk sent at the wrong offset is refused with the offset the service expects, so an
interrupted upload is resumed by calling ``upload_artifact`` again. A download writes to
``<path>.part`` with ``Range`` requests starting at what is already there and renames the
file once the digest matches.

Reference: packages/client/src/shadowspill_client/{artifacts.py, downloads.py} (resumable
transfers with digests).
"""
from __future__ import annotations

import hashlib
import os
from dataclasses import dataclass
from pathlib import Path

from .transport import HTTPTransport, TransportError

CHUNK_BYTES = 8 << 20


@dataclass(frozen=True)
class ArtifactHandle:
    artifact: str
    size: int
    sha256: str


def _digest(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        while True:
            block = f.read(1 << 20)
            if not block:
                return h.hexdigest()
            h.update(block)


def upload_artifact(transport: HTTPTransport, path: str | Path, *, name: str = "",
                    chunk_bytes: int = CHUNK_BYTES, on_progress=None) -> ArtifactHandle:
    path = Path(path)
    size, digest = path.stat().st_size, _digest(path)
    _, begun = transport.request("POST", "/v1/artifacts",
                                 {"name": name or path.name, "size": size, "sha256": digest})
    aid, offset = begun["artifact"], int(begun.get("received", 0))
    with open(path, "rb") as f:
        while offset < size:
            f.seek(offset)
            block = f.read(chunk_bytes)
            try:
                _, ack = transport.request("PUT", f"/v1/artifacts/{aid}/chunks/{offset}", block)
                offset = int(ack["received"])
            except TransportError as exc:
                if exc.status != 409:
                    raise
                # another attempt got further (or less far): ask where the service stands
                _, again = transport.request("POST", "/v1/artifacts",
                                             {"name": name or path.name, "size": size, "sha256": digest})
                offset = int(again["received"])
            if on_progress:
                on_progress(offset, size)
    transport.request("POST", f"/v1/artifacts/{aid}/complete", {})
    return ArtifactHandle(aid, size, digest)


def download_artifact(transport: HTTPTransport, artifact: str | ArtifactHandle, path: str | Path, *,
                      chunk_bytes: int = CHUNK_BYTES, on_progress=None) -> Path:
    aid = artifact.artifact if isinstance(artifact, ArtifactHandle) else artifact
    want = artifact.sha256 if isinstance(artifact, ArtifactHandle) else ""
    path = Path(path)
    part = path.with_name(path.name + ".part")
    have = part.stat().st_size if part.exists() else 0
    total = None
    with open(part, "ab") as f:
        while total is None or have < total:
            try:
                _, data = transport.request("GET", f"/v1/artifacts/{aid}", raw=True,
                                            headers={"Range": f"bytes={have}-{have + chunk_bytes - 1}"})
            except TransportError as exc:
                if exc.status == 416:        # nothing beyond what is here
                    break
                raise
            if not data:
                break
            f.write(data)
            have += len(data)
            if len(data) < chunk_bytes:
                total = have
            if on_progress:
                on_progress(have, total)
    if want and _digest(part) != want:
        part.unlink()
        raise IOError(f"artifact {aid}: digest mismatch after download")
    os.replace(part, path)
    return path


class PlansHandle:
    """The prepared plans of a run: what ``prepare_training`` / ``plan_training`` produce and what a
    later ``create_training_client(plans=...)`` starts from without preparing again.

    ``summary(page)`` lists the planned operations with their simulated times and traffic;
    ``save(name=)`` gives the plans a name inside the session; ``export(path)`` downloads the
    prepared bundle as a file, and ``ServiceClient.import_plans(path)`` uploads it to this or
    another service, whose new runs accept the returned handle as ``plans``. A bundle is reused
    only when its identity (model, geometry, budgets, frontend, dtype, world size) matches the new
    run's settings; otherwise the run prepares from scratch.
    Reference: packages/client/src/shadowspill_client/plans.py:26 (``PlansHandle``: ``report``,
    ``save``, ``summary``), preparation.py:29 (``PreparationHandle.export``)."""

    def __init__(self, service, run: str | None = None, artifact: ArtifactHandle | None = None):
        self._service, self.run, self.artifact = service, run, artifact

    def _route(self) -> str:
        if self.run is None:
            raise ValueError("these plans were imported as an artifact: they belong to no run of this service yet")
        return f"/v1/runs/{self._service.session}/{self.run}/plans"

    def summary(self, *, page: int = 0):
        if isinstance(page, bool) or not isinstance(page, int) or page < 0:
            raise ValueError("page must be a nonnegative int")
        route = self._route()
        return self._service.pool.submit(
            lambda: self._service.transport.request("GET", route, query={"page": page})[1])

    def save(self, *, name: str, operation: str = "step"):
        if not name or "/" in name:
            raise ValueError("a plan name is a non-empty string without '/'")
        route = self._route()
        return self._service.pool.submit(
            lambda: self._service.transport.request("POST", route, {"name": name, "plan": operation})[1])

    def named(self, name: str):
        """The plan a name was given to with ``save`` (its operation and summary)."""
        route = self._route()
        return self._service.pool.submit(
            lambda: self._service.transport.request("GET", route, query={"name": name})[1])

    def export(self, path, **kw):
        """Downloads the prepared bundle into ``path`` (a new file); the future gives the path."""
        route = self._route()

        def work():
            _, h = self._service.transport.request("POST", route + "/artifact", {})
            handle = ArtifactHandle(h["artifact"], int(h["size"]), h["sha256"])
            return download_artifact(self._service.transport, handle, path, **kw)
        return self._service.pool.submit(work)

    def create_arguments(self) -> dict:
        """What ``create_training_client`` sends for these plans."""
        return {"plans": self.run} if self.run is not None else {"plans_artifact": self.artifact.artifact}
