"""Node-level bookkeeping: device inventory, host/device admission leases, and
membership of node daemons through heartbeat-renewed leases on a monotonic clock.

A membership lease that expires fences the member permanently: a late heartbeat
from it is refused, it must join again under a new incarnation.
Reference: packages/engine/src/shadowspill/orchestration/{launch/device_inventory.py,
launch/admission.py, launch/host_arena.py, nodes/membership.py:28, nodes/registry.py}.
"""
from __future__ import annotations

import os
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, Callable

GIB = 1 << 30


def device_inventory() -> dict[str, Any]:
    """GPUs and host memory of this node (no CUDA context is created when torch is absent)."""
    gpus, names, device_gib = 0, [], 0.0
    try:
        import torch
        if torch.cuda.is_available():
            gpus = torch.cuda.device_count()
            for i in range(gpus):
                p = torch.cuda.get_device_properties(i)
                names.append(p.name)
                device_gib = p.total_memory / GIB
    except Exception:  # noqa: BLE001
        pass
    host_total = host_free = 0.0
    try:
        with open("/proc/meminfo") as f:
            info = {l.split(":")[0]: int(l.split()[1]) for l in f if ":" in l}
        host_total, host_free = info["MemTotal"] / (1 << 20), info.get("MemAvailable", 0) / (1 << 20)
    except OSError:
        pass
    inventory = {"gpus": gpus, "gpu_names": names, "device_gib": device_gib, "host_total_gib": host_total,
                 "host_free_gib": host_free, "cpus": os.cpu_count() or 1, "slurm_job": None}
    from . import slurm
    try:
        job = slurm.detect()
    except ValueError:
        job = None                       # a malformed Slurm environment offers the plain inventory
    return slurm.clamp_inventory(inventory, job, os.environ.get("SLURMD_NODENAME"))


class AdmissionError(RuntimeError):
    pass


class NodeAdmission:
    """Leases of device indices and host (pinned) bytes, so two runs never oversubscribe a node."""

    def __init__(self, gpus: int, host_bytes: int):
        self.gpus, self.host_bytes = gpus, host_bytes
        self._lock = threading.Lock()
        self._leases: dict[str, tuple[tuple[int, ...], int]] = {}

    def lease(self, n_gpus: int, host_bytes: int) -> tuple[str, tuple[int, ...]]:
        with self._lock:
            used = {g for gs, _ in self._leases.values() for g in gs}
            free = [g for g in range(self.gpus) if g not in used]
            held = sum(b for _, b in self._leases.values())
            if n_gpus > len(free):
                raise AdmissionError(f"{n_gpus} GPUs requested, {len(free)} free")
            if self.host_bytes and held + host_bytes > self.host_bytes:
                raise AdmissionError(f"host memory: {host_bytes / GIB:.1f} GiB requested, "
                                     f"{(self.host_bytes - held) / GIB:.1f} GiB free")
            lid = uuid.uuid4().hex
            self._leases[lid] = (tuple(free[:n_gpus]), host_bytes)
            return lid, tuple(free[:n_gpus])

    def release(self, lease_id: str) -> None:
        with self._lock:
            self._leases.pop(lease_id, None)

    def snapshot(self) -> dict[str, Any]:
        with self._lock:
            return {"leases": len(self._leases),
                    "gpus_used": sorted(g for gs, _ in self._leases.values() for g in gs),
                    "host_bytes_used": sum(b for _, b in self._leases.values())}


@dataclass
class Member:
    node_id: str
    incarnation: str
    expires: float
    info: dict[str, Any] = field(default_factory=dict)
    fenced: bool = False


class Membership:
    def __init__(self, lease_seconds: float = 15.0, clock: Callable[[], float] = time.monotonic):
        self.lease_seconds, self.clock = lease_seconds, clock
        self._lock = threading.Lock()
        self.members: dict[str, Member] = {}
        # commands for node daemons: delivered on poll until the daemon sends a receipt
        self._commands: dict[str, list[dict[str, Any]]] = {}

    def join(self, node_id: str, info: dict[str, Any] | None = None) -> str:
        with self._lock:
            inc = uuid.uuid4().hex
            self.members[node_id] = Member(node_id, inc, self.clock() + self.lease_seconds, info or {})
            return inc

    def heartbeat(self, node_id: str, incarnation: str) -> bool:
        with self._lock:
            m = self.members.get(node_id)
            now = self.clock()
            if m is None or m.incarnation != incarnation or m.fenced:
                return False
            if now > m.expires:
                m.fenced = True            # expiry fences permanently
                return False
            m.expires = now + self.lease_seconds
            return True

    def leave(self, node_id: str, incarnation: str) -> bool:
        with self._lock:
            m = self.members.get(node_id)
            if m is None or m.incarnation != incarnation:
                return False
            del self.members[node_id]
            return True

    def enqueue(self, node_id: str, command: dict[str, Any]) -> str:
        """Queues ``command`` for a live node's daemon; returns the command id."""
        with self._lock:
            m = self.members.get(node_id)
            if m is None or m.fenced or self.clock() > m.expires:
                raise KeyError(f"node {node_id!r} is not a live member")
            cid = uuid.uuid4().hex[:12]
            self._commands.setdefault(node_id, []).append(dict(command, id=cid, incarnation=m.incarnation))
            return cid

    def poll(self, node_id: str, incarnation: str) -> list[dict[str, Any]] | None:
        """A daemon's poll renews its lease and returns every command it has not acknowledged
        (at-least-once delivery); ``None`` for a fenced or unknown incarnation."""
        if not self.heartbeat(node_id, incarnation):
            return None
        with self._lock:
            return [c for c in self._commands.get(node_id, []) if c["incarnation"] == incarnation]

    def receipt(self, node_id: str, incarnation: str, command_id: str, outcome: dict[str, Any] | None = None) -> bool:
        """Acknowledges one command; it is not delivered again. False if unknown."""
        with self._lock:
            m = self.members.get(node_id)
            if m is None or m.incarnation != incarnation:
                return False
            queue = self._commands.get(node_id, [])
            for i, c in enumerate(queue):
                if c["id"] == command_id:
                    del queue[i]
                    m.info.setdefault("receipts", []).append({"id": command_id, **(outcome or {})})
                    return True
            return False

    def reconcile(self) -> list[str]:
        """Fences every member whose lease ran out; returns their ids."""
        with self._lock:
            now = self.clock()
            lost = [m.node_id for m in self.members.values() if not m.fenced and now > m.expires]
            for n in lost:
                self.members[n].fenced = True
            return lost

    def live(self) -> list[str]:
        with self._lock:
            now = self.clock()
            return sorted(m.node_id for m in self.members.values() if not m.fenced and now <= m.expires)
