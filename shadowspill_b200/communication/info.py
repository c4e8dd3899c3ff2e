"""Measured link facts the planner and simulator consume.

``CommunicationInfo`` carries the host-link rates of one worker (fetch = spill
to device, evict = device to spill, each alone and with the other direction in
flight), their latencies, and the measured costs of the collectives a plan
uses. It corresponds to the reference's ``CommunicationInfo``
(packages/engine/src/shadowspill/communication/info.py:15); the default rates
are a PCIe Gen5 x16 host link as calibrated on H100/B200-class hosts
(about 52 GB/s each way) and NVLink 5 peer rates measured on B200.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Any


@dataclass
class CommunicationInfo:
    fetch_solo_bps: float = 52e9
    fetch_concurrent_bps: float = 48e9
    evict_solo_bps: float = 50e9
    evict_concurrent_bps: float = 46e9
    fetch_latency_ns: int = 8_000
    evict_latency_ns: int = 8_000
    scale_up_bps: float = 770e9          # NVLink peer copy, per direction per GPU
    scale_up_latency_ns: int = 6_000
    scale_out_bps: float = 50e9
    scale_out_latency_ns: int = 20_000
    world_size: int = 1
    collectives: dict[str, float] = field(default_factory=dict)   # "op:ranks:bytes" -> seconds
    backend: dict[str, Any] = field(default_factory=dict)
    source: str = "default"

    def to_json(self) -> dict[str, Any]:
        return asdict(self)

    @staticmethod
    def from_json(d: dict[str, Any]) -> "CommunicationInfo":
        return CommunicationInfo(**d)

    def collective_seconds(self, op: str, ranks: int, nbytes: int) -> float:
        """Measured cost when this exact (op, ranks, bytes) was calibrated, else a
        flat-ring estimate ``factor*(n-1)*(latency + chunk/bandwidth)``
        (reference: communication/collectives.py:107-175)."""
        key = f"{op}:{ranks}:{nbytes}"
        if key in self.collectives:
            return self.collectives[key]
        if ranks <= 1 or nbytes <= 0:
            return 0.0
        factor = 2.0 if op == "all_reduce" else 1.0
        chunk = nbytes / ranks
        return factor * (ranks - 1) * (self.scale_up_latency_ns * 1e-9 + chunk / self.scale_up_bps)
