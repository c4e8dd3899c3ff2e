"""Checkpoint archive: an uncompressed GNU TAR of raw tensor members followed by
``manifest.json`` and ``manifest.blake3``.

Layout (the reference's, packages/engine/src/shadowspill/checkpoint/archive.py:39-61
and save.py:263-291): members ``tensors/<i>`` hold the little-endian bytes of the
region of tensor *i* this logical rank owns, each padded to 512 bytes by TAR;
``manifest.json`` describes them; ``manifest.blake3`` is the BLAKE3 hex digest of
the manifest bytes; two zero blocks end the archive. One archive per logical
rank, written to a temporary name, fsynced, renamed, directory fsynced.
"""
from __future__ import annotations

import io
import json
import os
import tarfile
from pathlib import Path
from typing import Any, Iterator

import numpy as np

from ..native import Blake3

FORMAT = "shadowspill.checkpoint"
VERSION = 1
CHUNK = 64 << 20           # bytes hashed and written per slice


class CheckpointError(RuntimeError):
    pass


class _HashingReader(io.RawIOBase):
    """File-like view of a byte buffer that hashes what tarfile reads from it."""

    def __init__(self, buf: memoryview):
        self.buf, self.pos, self.hasher = buf, 0, Blake3()

    def readable(self) -> bool:
        return True

    def read(self, n: int = -1) -> bytes:
        if n < 0 or n > len(self.buf) - self.pos:
            n = len(self.buf) - self.pos
        n = min(n, CHUNK)
        chunk = self.buf[self.pos:self.pos + n]
        self.pos += n
        self.hasher.update(chunk)
        return bytes(chunk)


class ArchiveWriter:
    def __init__(self, path: str | Path):
        self.path = Path(path)
        self.tmp = self.path.with_name(self.path.name + ".partial")
        self.path.parent.mkdir(parents=True, exist_ok=True)
        self.file = open(self.tmp, "wb")
        self.tar = tarfile.open(fileobj=self.file, mode="w", format=tarfile.GNU_FORMAT)
        self.entries: list[dict[str, Any]] = []

    def add_tensor(self, entry: dict[str, Any], data: np.ndarray) -> None:
        """``data`` is the contiguous owned region as raw bytes (uint8 view)."""
        member = f"tensors/{len(self.entries)}"
        raw = memoryview(np.ascontiguousarray(data).view(np.uint8).reshape(-1))
        info = tarfile.TarInfo(member)
        info.size = len(raw)
        info.mtime = 0
        reader = _HashingReader(raw)
        self.tar.addfile(info, reader)
        entry = dict(entry, member=member, bytes=len(raw), blake3=reader.hasher.hexdigest())
        self.entries.append(entry)

    def finish(self, manifest: dict[str, Any]) -> Path:
        manifest = dict(manifest, tensors=self.entries)
        blob = json.dumps(manifest, sort_keys=True, separators=(",", ":")).encode()
        for name, payload in (("manifest.json", blob),
                              ("manifest.blake3", Blake3(blob).hexdigest().encode())):
            info = tarfile.TarInfo(name)
            info.size = len(payload)
            info.mtime = 0
            self.tar.addfile(info, io.BytesIO(payload))
        self.tar.close()                 # writes the two zero blocks
        self.file.flush()
        os.fsync(self.file.fileno())
        self.file.close()
        os.replace(self.tmp, self.path)
        dirfd = os.open(self.path.parent, os.O_RDONLY)
        try:
            os.fsync(dirfd)
        finally:
            os.close(dirfd)
        return self.path

    def abort(self) -> None:
        try:
            self.tar.close()
            self.file.close()
        finally:
            self.tmp.unlink(missing_ok=True)


def read_manifest(path: str | Path) -> dict[str, Any]:
    with tarfile.open(path, "r:") as tar:
        try:
            blob = tar.extractfile("manifest.json").read()
            seal = tar.extractfile("manifest.blake3").read().decode().strip()
        except KeyError as exc:
            raise CheckpointError(f"{path}: incomplete archive ({exc})") from None
    if Blake3(blob).hexdigest() != seal:
        raise CheckpointError(f"{path}: manifest does not match its BLAKE3 seal")
    manifest = json.loads(blob)
    if manifest.get("format") != FORMAT:
        raise CheckpointError(f"{path}: not a {FORMAT} archive")
    if manifest.get("version") != VERSION:
        raise CheckpointError(f"{path}: unsupported checkpoint version {manifest.get('version')}")
    return manifest


def iter_members(path: str | Path, verify: bool = True) -> Iterator[tuple[dict[str, Any], np.ndarray]]:
    """Yields ``(entry, uint8 array)`` for every tensor member, checking digests."""
    manifest = read_manifest(path)
    with tarfile.open(path, "r:") as tar:
        for entry in manifest["tensors"]:
            f = tar.extractfile(entry["member"])
            data = np.frombuffer(f.read(), dtype=np.uint8)
            if data.nbytes != entry["bytes"]:
                raise CheckpointError(f"{path}: {entry['member']} is truncated")
            if verify and Blake3(data.tobytes()).hexdigest() != entry["blake3"]:
                raise CheckpointError(f"{path}: {entry['name']} fails its BLAKE3 check")
            yield entry, data
