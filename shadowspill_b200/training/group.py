"""Worker group: launches one worker process per rank and runs two-phase commands.

``execute`` sends the call to every rank, waits until all are ``ready`` (inputs
staged and validated), then tells all to ``execute``; if any rank fails to stage,
every rank is told to ``abort`` and training state is untouched. A failure after
execution began marks the whole group's state invalid.
Reference: packages/engine/src/shadowspill/training/worker/{group.py:54-99,launch.py:28,startup.py:71}.
"""
from __future__ import annotations

import os
import socket
import subprocess
import sys
import threading
from pathlib import Path

from .channel import Channel, ChannelClosed


class WorkerFailure(RuntimeError):
    def __init__(self, message: str, effect: str = "unknown"):
        self.effect = effect
        super().__init__(message)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class BoundedLog(threading.Thread):
    """Copies a worker's output into its log file up to ``limit`` bytes, says once that the limit
    was reached, and keeps draining the pipe after that so that a chatty worker never blocks on a
    full pipe or fills the service's disk. (The reference bounds its worker logs the same way:
    packages/engine/src/shadowspill/orchestration/launch/log_files.py.)"""

    def __init__(self, stream, path, limit: int):
        super().__init__(daemon=True, name=f"worker-log:{Path(path).name}")
        self.stream, self.path, self.limit = stream, Path(path), max(1024, int(limit))
        self.written = self.path.stat().st_size if self.path.exists() else 0
        self.dropped = 0

    def run(self) -> None:
        noted = False
        with open(self.path, "ab", buffering=0) as out:
            while True:
                block = self.stream.read1(65536) if hasattr(self.stream, "read1") else self.stream.read(65536)
                if not block:
                    break
                room = self.limit - self.written
                if room > 0:
                    out.write(block[:room])
                    self.written += min(room, len(block))
                if len(block) > max(room, 0):
                    self.dropped += len(block) - max(room, 0)
                    if not noted:
                        out.write(f"\n[log limit of {self.limit} bytes reached; later output is dropped]\n".encode())
                        noted = True
        try:
            self.stream.close()
        except OSError:
            pass


class WorkerGroup:
    def __init__(self, setups: list[dict], log_dir: str | Path, checkpoint: str | None = None,
                 startup_seconds: float = 1800.0, on_progress=None):
        self.world = len(setups)
        self.log_dir = Path(log_dir)
        self.log_dir.mkdir(parents=True, exist_ok=True)
        self.procs: list[subprocess.Popen] = []
        self.chans: list[Channel] = []
        self.valid = True
        self.ready_info: list[dict] = []
        self.on_progress = on_progress or (lambda msg: None)
        port = _free_port()
        root = str(Path(__file__).resolve().parents[2])
        for rank, setup in enumerate(setups):
            to_child_r, to_child_w = os.pipe()
            from_child_r, from_child_w = os.pipe()
            env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
            limit = int(setup.get("max_worker_log_bytes") or os.environ.get("SHADOWSPILL_WORKER_LOG_BYTES", 64 << 20))
            command = [sys.executable, "-m", "shadowspill_b200.training.worker", "--control-fd",
                       f"{to_child_r},{from_child_w}"]
            from ..orchestration import capture
            nsys = capture.NsysOptions.from_json(setup.get("nsys"))
            if nsys is not None and capture.available(nsys):
                command = capture.wrap_command(command, rank, self.log_dir, nsys)
            elif nsys is not None:
                self.on_progress(f"[rank={rank}] nsys capture requested but {nsys.executable} is not "
                                 f"installed; running unprofiled")
            proc = subprocess.Popen(command, pass_fds=(to_child_r, from_child_w), env=env,
                                    stdout=subprocess.PIPE, stderr=subprocess.STDOUT, cwd=root)
            BoundedLog(proc.stdout, self.log_dir / f"worker{rank}.log", limit).start()
            os.close(to_child_r); os.close(from_child_w)
            chan = Channel(from_child_r, to_child_w)
            chan.send({"type": "launch", "rank": rank, "world_size": self.world, "setup": setup,
                       "master_addr": "127.0.0.1", "master_port": port, "checkpoint": checkpoint})
            self.procs.append(proc)
            self.chans.append(chan)
        try:
            for rank, chan in enumerate(self.chans):
                self.ready_info.append(self._await(rank, chan, "ready", startup_seconds))
        except BaseException:
            self.stop()
            raise

    def _await(self, rank: int, chan: Channel, want: str, timeout: float | None) -> dict:
        while True:
            try:
                header, _ = chan.recv(timeout)
            except (ChannelClosed, TimeoutError) as exc:
                self.valid = False
                raise WorkerFailure(f"worker {rank} lost: {exc}") from None
            kind = header.get("type")
            if kind == "progress":
                self.on_progress(f"[rank={rank}] {header.get('message', '')}")
                continue
            if kind == "failed":
                raise WorkerFailure(f"worker {rank} failed to start: {header.get('error')}\n"
                                    f"{header.get('traceback', '')}", "not_started")
            if kind == want or kind == "reply":
                return header

    def execute(self, request_id: str, operation: str, arguments: dict,
                payloads: list[bytes] | None = None, timeout: float | None = None) -> list[dict]:
        if not self.valid:
            if operation == "close":
                # nothing to run on state of unknown content: the caller tears the workers down
                return [{"state": "completed", "outputs": {}} for _ in self.chans]
            raise WorkerFailure("training state is invalid after an earlier failure; only close "
                                "is accepted", "not_started")
        for rank, chan in enumerate(self.chans):
            chan.send({"type": "call", "request_id": request_id, "operation": operation,
                       "arguments": arguments}, payloads[rank] if payloads else b"")
        staged = [self._await(r, c, "reply", timeout) for r, c in enumerate(self.chans)]
        bad = [s for s in staged if s.get("state") != "ready"]
        action = "abort" if bad else "execute"
        for chan in self.chans:
            chan.send({"type": "control", "request_id": request_id, "action": action})
        replies = [self._await(r, c, "reply", timeout) for r, c in enumerate(self.chans)]
        if bad:
            raise WorkerFailure(f"staging failed: {bad[0].get('error')}", "not_started")
        failed = [r for r in replies if r.get("state") != "completed"]
        if failed:
            effect = "unknown" if any(r.get("effect") == "unknown" for r in failed) else "not_started"
            if effect == "unknown":
                self.valid = False
            raise WorkerFailure(f"{failed[0].get('error')}\n{failed[0].get('traceback', '')}", effect)
        return replies

    def stop(self) -> None:
        for chan in self.chans:
            try:
                chan.send({"type": "shutdown"})
            except ChannelClosed:
                pass
        from ..parallel.collectives import nvls_requested
        for proc in self.procs:
            try:
                proc.wait(timeout=30)
            except subprocess.TimeoutExpired:
                if nvls_requested():
                    # memory bound to an NVSwitch multicast object: a killed rank can fault its
                    # peers' GPUs, so wait for the rank to leave between steps on its own
                    proc.wait()
                else:
                    proc.kill()
        for chan in self.chans:
            chan.close()
        self.procs, self.chans = [], []
