"""Pipeline results as single archive files.

An archive is a ZIP of data only: ``manifest.json`` (format, kind, version,
payload table), ``metadata.json`` (the artifact's JSON value) and binary
payloads stored once each under ``payloads/<sha256>``. Saving writes a
temporary file beside the destination, fsyncs it, renames it over the
destination and fsyncs the directory, so a crash leaves either the old or the
new archive. Loading verifies every payload against its SHA-256 and runs
nothing from the file.

Kinds: ``program``, ``profiles``, ``plan``, ``sweep``, ``budgets``,
``communication``, ``pool_memory``, ``tensor_chunk``. Same contract as the
reference's archives (packages/engine/src/shadowspill/artifacts/archive.py:20-140;
tensors.py:54-72 for tensor chunks).
"""
from __future__ import annotations

import hashlib
import json
import os
import tempfile
import zipfile
from pathlib import Path
from typing import Any, Mapping

FORMAT = "ss-b200.artifact"
VERSION = 1


class ArtifactError(ValueError):
    pass


def _fsync_dir(path: Path) -> None:
    fd = os.open(path, os.O_RDONLY)
    try:
        os.fsync(fd)
    finally:
        os.close(fd)


def save_archive(path: str | os.PathLike, kind: str, metadata: Mapping[str, Any],
                 payloads: Mapping[str, bytes] | None = None, max_bytes: int | None = None) -> Path:
    """``payloads`` maps a logical name to bytes; equal contents are stored once."""
    if max_bytes is not None and (type(max_bytes) is not int or max_bytes < 0):
        raise ValueError("archive byte limit must be a non-negative integer")
    dest = Path(path)
    dest.parent.mkdir(parents=True, exist_ok=True)
    payloads = dict(payloads or {})
    table = {name: {"sha256": hashlib.sha256(data).hexdigest(), "bytes": len(data)}
             for name, data in payloads.items()}
    manifest = {"format": FORMAT, "version": VERSION, "kind": kind, "payloads": table}
    fd, tmp = tempfile.mkstemp(prefix=dest.name + ".", suffix=".tmp", dir=dest.parent)
    try:
        with os.fdopen(fd, "wb") as f:
            with zipfile.ZipFile(f, "w", zipfile.ZIP_STORED) as z:
                z.writestr("manifest.json", json.dumps(manifest, sort_keys=True))
                z.writestr("metadata.json", json.dumps(metadata, sort_keys=True))
                written = set()
                for name, data in payloads.items():
                    digest = table[name]["sha256"]
                    if digest not in written:
                        z.writestr(f"payloads/{digest}", data)
                        written.add(digest)
            f.flush()
            if max_bytes is not None and f.tell() > max_bytes:
                raise ArtifactError(f"archive is {f.tell()} bytes, limit {max_bytes}")
            os.fsync(f.fileno())
        os.replace(tmp, dest)
        _fsync_dir(dest.parent)
    except BaseException:
        try:
            os.unlink(tmp)
        except FileNotFoundError:
            pass
        raise
    return dest


def load_archive(path: str | os.PathLike, kind: str | None = None) -> tuple[dict, dict[str, bytes]]:
    """Returns ``(metadata, payloads by logical name)``; raises ``ArtifactError`` on a wrong
    kind, an unknown format or a payload whose bytes do not match its digest."""
    with zipfile.ZipFile(path, "r") as z:
        try:
            manifest = json.loads(z.read("manifest.json"))
            metadata = json.loads(z.read("metadata.json"))
        except KeyError as exc:
            raise ArtifactError(f"not an artifact archive: {exc}") from None
        if manifest.get("format") != FORMAT or manifest.get("version") != VERSION:
            raise ArtifactError("unknown artifact format or version")
        if kind is not None and manifest.get("kind") != kind:
            raise ArtifactError(f"archive holds a {manifest.get('kind')!r}, wanted {kind!r}")
        blobs: dict[str, bytes] = {}
        out: dict[str, bytes] = {}
        for name, entry in manifest.get("payloads", {}).items():
            digest = entry["sha256"]
            if digest not in blobs:
                data = z.read(f"payloads/{digest}")
                if hashlib.sha256(data).hexdigest() != digest or len(data) != entry["bytes"]:
                    raise ArtifactError(f"payload {name!r} does not match its digest")
                blobs[digest] = data
            out[name] = blobs[digest]
    return metadata, out


def archive_kind(path: str | os.PathLike) -> str:
    with zipfile.ZipFile(path, "r") as z:
        return json.loads(z.read("manifest.json")).get("kind", "")
