"""The reference client's control protocol, as far as this server answers it.

The reference client (packages/client/src/shadowspill_client/transport/http.py:228 ``_start``,
:257 ``_metadata``) sends ``Accept: application/vnd.shadowspill.control+json`` with every request and
accepts only replies of that media type whose body is the envelope ``{"version": 1, "kind": ...,
"value": {...}}`` (protocol/codec.py:204) with a record kind from its fixed allowlist; an
unsuccessful reply must carry a ``service.error`` record. This module produces those envelopes for
the connection-level records (``service.info``, ``service.hardware``, ``service.error``), so that
the unmodified reference client connects to this server, authenticates and lists hardware. The
training records (setup, preview, run, request, metric, checkpoint and plan pages: some fifty
kinds) are not translated: a reference-protocol request to any other route gets a ``service.error``
with code ``unsupported`` that names the route, instead of a body the client would reject as
malformed. This framework's own client (``shadowspill_b200.client``) speaks plain JSON records on
the same routes.
"""
from __future__ import annotations

import json
import re
from typing import Any

CONTROL_MEDIA_TYPE = "application/vnd.shadowspill.control+json"
VERSION = 1
GIB = 1 << 30

_IDENT = re.compile(r"[^A-Za-z0-9_.:-]")


def wants_control(headers) -> bool:
    return (headers.get("Accept") or "").strip() == CONTROL_MEDIA_TYPE


def envelope(kind: str, value: dict[str, Any]) -> bytes:
    return json.dumps({"version": VERSION, "kind": kind, "value": value}, sort_keys=True,
                      separators=(",", ":"), allow_nan=False).encode()


def identifier(text: str, fallback: str = "x") -> str:
    """An opaque identifier in the reference's alphabet (protocol/requests.py:22)."""
    out = _IDENT.sub("-", str(text))[:128].lstrip("_.:-")
    return out or fallback


def service_info(incarnation: str, owner: str) -> bytes:
    return envelope("service.info", {"server_incarnation": identifier(incarnation, "incarnation"),
                                     "owner_id": identifier(owner, "local")})


def service_error(status: int, message: str) -> bytes:
    code = {400: "invalid_request", 401: "unauthenticated", 403: "forbidden", 404: "not_found",
            409: "conflict", 413: "too_large", 429: "backpressure", 501: "unsupported",
            503: "unavailable"}.get(status, "internal")
    return envelope("service.error", {"code": code, "message": str(message)[:1024] or code})


def hardware_inventory(hardware: dict[str, Any], admission: dict[str, Any], node_id: str = "local",
                       pool: str = "default") -> bytes:
    """``service.hardware``: one node with its devices (protocol/hardware.py:14,48,97)."""
    used = set(admission.get("gpus_used", ()))
    names = list(hardware.get("gpu_names") or [])
    capacity = max(1, int(float(hardware.get("device_gib") or 0) * GIB))
    devices = [{"id": f"{node_id}:gpu{i}", "index": i, "gpu_type": names[i] if i < len(names) else None,
                "capacity_bytes": capacity, "available": i not in used}
               for i in range(int(hardware.get("gpus") or 0))]
    host_capacity = int(float(hardware.get("host_total_gib") or 0) * GIB)
    host_available = max(0, min(host_capacity, int(float(hardware.get("host_free_gib") or 0) * GIB)
                                - int(admission.get("host_bytes_used", 0))))
    node = {"id": node_id, "pool": pool, "devices": devices, "host_capacity_bytes": host_capacity,
            "host_available_bytes": host_available, "cpu_count": max(1, int(hardware.get("cpus") or 1)),
            "driver": None}
    return envelope("service.hardware", {"nodes": [node]})
