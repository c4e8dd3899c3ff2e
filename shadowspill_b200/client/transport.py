"""HTTP(S) transport with bounded request bodies, and an SSH tunnel helper.

Reference: packages/client/src/shadowspill_client/transport/{http,ssh}.py.
"""
from __future__ import annotations

import http.client
import json
import os
import re
import signal
import socket
import subprocess
import time
import urllib.parse
from dataclasses import dataclass
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


_DESTINATION = re.compile(r"[A-Za-z0-9_.@:%+\[\],-]{1,1024}")
_SERVER = re.compile(r"[A-Za-z0-9_.:%-]{1,253}")


@dataclass(frozen=True)
class SSH:
    """How to reach a service through OpenSSH (``ServiceClient(url=None, ssh=SSH(...))``).

    ``host`` is an OpenSSH destination or alias; keys, agents, jump hosts and control masters come
    from the OpenSSH configuration (``config_file`` names another one). ``server_host`` /
    ``server_port`` say where the service listens as seen from ``host``. The client forwards a
    local port and never prompts, so authentication has to work non-interactively. These settings
    stay on this machine: nothing of them is sent to the service or saved with a run.
    Reference: packages/client/src/shadowspill_client/transport/ssh.py:24 (``SSH``)."""
    host: str
    server_port: int
    server_host: str = "127.0.0.1"
    jump_host: str | None = None
    ssh_port: int | None = None
    config_file: str | None = None

    def __post_init__(self):
        for name in ("host", "jump_host"):
            value = getattr(self, name)
            if value is None and name == "jump_host":
                continue
            if not isinstance(value, str) or not _DESTINATION.fullmatch(value) or value.startswith("-"):
                raise ValueError(f"{name} must be an OpenSSH destination or alias")
        if not isinstance(self.server_host, str) or not _SERVER.fullmatch(self.server_host):
            raise ValueError("server_host must be a host name or an IP address")
        for name in ("server_port", "ssh_port"):
            value = getattr(self, name)
            if value is None and name == "ssh_port":
                continue
            if isinstance(value, bool) or not isinstance(value, int) or not 1 <= value <= 65535:
                raise ValueError(f"{name} must be a port number")
        if self.config_file is not None and (not isinstance(self.config_file, str) or not self.config_file
                                             or "\0" in self.config_file):
            raise ValueError("config_file must be a path")

    def command(self, local_port: int, executable: str = "ssh") -> list[str]:
        """The OpenSSH invocation that holds the forward open in the foreground."""
        cmd = [executable, "-N", "-T", "-o", "BatchMode=yes", "-o", "ExitOnForwardFailure=yes",
               "-o", "ServerAliveInterval=15", "-o", "ServerAliveCountMax=4"]
        if self.config_file:
            cmd += ["-F", self.config_file]
        if self.jump_host:
            cmd += ["-J", self.jump_host]
        if self.ssh_port:
            cmd += ["-p", str(self.ssh_port)]
        cmd += ["-L", f"127.0.0.1:{local_port}:{self.server_host}:{self.server_port}", "--", self.host]
        return cmd


class SSHTunnel:
    """One owned local forward to a service. ``open()`` (or entering the context) starts OpenSSH in
    its own process group and waits until the local port accepts connections; it confirms the
    forward only, the caller still authenticates to the service over it. ``close()`` ends the
    process group; there is no reconnect and nothing is retried. The older positional form
    ``SSHTunnel(host, remote_port, user=, local_port=)`` is kept."""

    def __init__(self, settings, remote_port: int | None = None, user: str = "", local_port: int = 0,
                 timeout: float = 30.0, executable: str | None = None):
        if not isinstance(settings, SSH):
            settings = SSH(f"{user}@{settings}" if user else settings, int(remote_port))
        if not 0 < timeout <= 300:
            raise ValueError("the connection timeout must be in (0, 300] seconds")
        self.settings, self.timeout = settings, float(timeout)
        self.executable = executable or os.environ.get("SHADOWSPILL_SSH", "ssh")
        self.local_port = local_port or self._free_port()
        self.proc: subprocess.Popen | None = None
        self.closed = False

    @staticmethod
    def _free_port() -> int:
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            return s.getsockname()[1]

    @property
    def url(self) -> str:
        return f"http://127.0.0.1:{self.local_port}"

    def open(self) -> str:
        if self.proc is not None:
            return self.url
        self.proc = subprocess.Popen(self.settings.command(self.local_port, self.executable),
                                     stdin=subprocess.DEVNULL, stdout=subprocess.DEVNULL,
                                     stderr=subprocess.PIPE, start_new_session=True)
        deadline = time.monotonic() + self.timeout
        while time.monotonic() < deadline:
            if self.proc.poll() is not None:
                err = (self.proc.stderr.read() or b"").decode(errors="replace").strip().splitlines()
                status, self.proc = self.proc.returncode, None
                raise ConnectionError("ssh exited before the forward came up"
                                      + (f": {err[-1]}" if err else f" (status {status})"))
            with socket.socket() as s:
                s.settimeout(0.5)
                if s.connect_ex(("127.0.0.1", self.local_port)) == 0:
                    return self.url
            time.sleep(0.1)
        self.close()
        raise TimeoutError(f"the ssh forward to {self.settings.host} did not come up in {self.timeout:g} s")

    def close(self) -> None:
        proc, self.proc = self.proc, None
        self.closed = True
        if proc is None or proc.poll() is not None:
            return
        try:
            os.killpg(proc.pid, signal.SIGTERM)          # the process group this tunnel started, nothing else
        except (ProcessLookupError, PermissionError):
            proc.terminate()
        try:
            proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            try:
                os.killpg(proc.pid, signal.SIGKILL)
            except (ProcessLookupError, PermissionError):
                proc.kill()
            proc.wait(timeout=5)

    def __enter__(self) -> str:
        return self.open()

    def __exit__(self, *exc):
        self.close()
