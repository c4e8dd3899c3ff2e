"""HTTP(S) transport with bounded request bodies, and an SSH tunnel helper.

Reference: packages/client/src/shadowspill_client/transport/{http,ssh}.py.
"""
from __future__ import annotations

import http.client
import json
import socket
import subprocess
import time
import urllib.parse
from typing import Any


class TransportError(RuntimeError):
    def __init__(self, status: int, message: str):
        self.status = status
        super().__init__(f"HTTP {status}: {message}")


class HTTPTransport:
    def __init__(self, url: str, token: str = "", timeout: float = 600.0):
        u = urllib.parse.urlparse(url if "://" in url else "http://" + url)
        self.secure = u.scheme == "https"
        self.host, self.port = u.hostname or "127.0.0.1", u.port or (443 if self.secure else 80)
        self.token, self.timeout = token, timeout

    def _conn(self):
        cls = http.client.HTTPSConnection if self.secure else http.client.HTTPConnection
        return cls(self.host, self.port, timeout=self.timeout)

    def request(self, method: str, path: str, body: bytes | dict | None = None,
                query: dict[str, Any] | None = None, raw: bool = False,
                headers: dict[str, str] | None = None):
        headers = dict(headers or {})
        if self.token:
            headers["Authorization"] = f"Bearer {self.token}"
        if isinstance(body, dict):
            body = json.dumps(body).encode()
            headers["Content-Type"] = "application/json"
        elif body is not None:
            headers["Content-Type"] = "application/octet-stream"
        if query:
            path += "?" + urllib.parse.urlencode(query)
        conn = self._conn()
        try:
            conn.request(method, path, body=body, headers=headers)
            resp = conn.getresponse()
            data = resp.read()
        finally:
            conn.close()
        if resp.status >= 400:
            try:
                msg = json.loads(data).get("error", data.decode(errors="replace"))
            except Exception:  # noqa: BLE001
                msg = data.decode(errors="replace")
            raise TransportError(resp.status, msg)
        if raw:
            return resp.status, data
        return resp.status, (json.loads(data) if data else {})


class SSHTunnel:
    """``ssh -N -L`` to a remote service; context manager yielding a local URL."""

    def __init__(self, host: str, remote_port: int, user: str = "", local_port: int = 0):
        self.target = f"{user}@{host}" if user else host
        self.remote_port = remote_port
        self.local_port = local_port or self._free_port()
        self.proc: subprocess.Popen | None = None

    @staticmethod
    def _free_port() -> int:
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            return s.getsockname()[1]

    def __enter__(self) -> str:
        self.proc = subprocess.Popen(["ssh", "-N", "-o", "ExitOnForwardFailure=yes", "-L",
                                      f"{self.local_port}:127.0.0.1:{self.remote_port}", self.target])
        deadline = time.monotonic() + 30
        while time.monotonic() < deadline:
            if self.proc.poll() is not None:
                raise RuntimeError("ssh tunnel exited")
            with socket.socket() as s:
                if s.connect_ex(("127.0.0.1", self.local_port)) == 0:
                    return f"http://127.0.0.1:{self.local_port}"
            time.sleep(0.2)
        raise TimeoutError("ssh tunnel did not come up")

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
