"""Length-prefixed typed frames over a pair of inherited file descriptors.

The service talks to each worker through a private channel (two pipes whose fds
the child inherits), never through the worker's stdout, so log output cannot
corrupt the protocol. A frame is ``[8-byte length][JSON header][payload]``.
Reference: packages/engine/src/shadowspill/training/worker/channel.py.
"""
from __future__ import annotations

import json
import os
import select
import struct


class ChannelClosed(ConnectionError):
    pass


class Channel:
    def __init__(self, read_fd: int, write_fd: int):
        self.r, self.w = read_fd, write_fd

    def send(self, header: dict, payload: bytes = b"") -> None:
        head = json.dumps(header).encode()
        blob = struct.pack(">QQ", len(head), len(payload)) + head + payload
        view = memoryview(blob)
        while view:
            try:
                n = os.write(self.w, view[:1 << 20])
            except (BrokenPipeError, OSError) as exc:
                raise ChannelClosed(str(exc)) from None
            view = view[n:]

    def _read(self, n: int, timeout: float | None) -> bytes:
        out = bytearray()
        while len(out) < n:
            if timeout is not None:
                ready, _, _ = select.select([self.r], [], [], timeout)
                if not ready:
                    raise TimeoutError("worker channel timed out")
            chunk = os.read(self.r, min(n - len(out), 1 << 20))
            if not chunk:
                raise ChannelClosed("peer closed the channel")
            out += chunk
        return bytes(out)

    def recv(self, timeout: float | None = None) -> tuple[dict, bytes]:
        hl, pl = struct.unpack(">QQ", self._read(16, timeout))
        header = json.loads(self._read(hl, timeout))
        payload = self._read(pl, timeout) if pl else b""
        return header, payload

    def close(self) -> None:
        for fd in (self.r, self.w):
            try:
                os.close(fd)
            except OSError:
                pass
