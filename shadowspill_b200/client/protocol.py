"""Wire protocol: typed records plus binary payload framing.

A message is ``[8-byte big-endian header length][JSON header][payload bytes]``;
arrays travel as raw little-endian bytes described in the header. Records mirror
the reference's request/result/run records
(packages/client/src/shadowspill_client/protocol/{requests,results,codec}.py).
"""
from __future__ import annotations

import hashlib
import json
import struct
import uuid
from dataclasses import asdict, dataclass, field
from typing import Any

import numpy as np

OPERATIONS = ("step", "forward_backward", "forward", "optim_step", "discard", "save", "restore",
              "export", "plan_report", "close")


@dataclass
class OperationRequest:
    operation: str
    request_id: str = ""
    dependencies: list[str] = field(default_factory=list)
    arguments: dict[str, Any] = field(default_factory=dict)
    has_input: bool = False
    writer_id: str = ""

    def __post_init__(self):
        if self.operation not in OPERATIONS:
            raise ValueError(f"unknown operation {self.operation!r}")
        if not self.request_id:
            self.request_id = uuid.uuid4().hex

    def digest(self) -> str:
        body = {"operation": self.operation, "request_id": self.request_id,
                "dependencies": self.dependencies, "arguments": self.arguments}
        return hashlib.sha256(json.dumps(body, sort_keys=True).encode()).hexdigest()


@dataclass
class OperationResult:
    request_id: str
    state: str                         # pending | running | completed | failed | rejected
    effect: str = "not_started"        # not_started | completed | unknown
    loss: float | None = None
    metrics: dict[str, float] = field(default_factory=dict)
    completed_updates: int = 0
    execution_seconds: float = 0.0
    error: str = ""
    outputs: dict[str, Any] = field(default_factory=dict)

    @property
    def done(self) -> bool:
        return self.state in ("completed", "failed", "rejected")


@dataclass
class RunInfo:
    session: str
    run: str
    state: str                         # preparing | ready | failed | closed
    workers: int = 0
    plan_summary: dict[str, Any] = field(default_factory=dict)
    error: str = ""
    state_valid: bool = True


def to_json(rec) -> dict[str, Any]:
    return asdict(rec)


def encode_arrays(header: dict[str, Any], arrays: dict[str, np.ndarray]) -> bytes:
    """Frames a JSON header and named arrays into one message."""
    specs, chunks, off = [], [], 0
    for name, a in arrays.items():
        a = np.ascontiguousarray(a)
        raw = a.tobytes()
        specs.append({"name": name, "dtype": a.dtype.str, "shape": list(a.shape), "offset": off,
                      "bytes": len(raw)})
        chunks.append(raw)
        off += len(raw)
    head = json.dumps(dict(header, arrays=specs)).encode()
    return struct.pack(">Q", len(head)) + head + b"".join(chunks)


def decode_arrays(blob: bytes) -> tuple[dict[str, Any], dict[str, np.ndarray]]:
    if len(blob) < 8:
        raise ValueError("truncated message")
    (n,) = struct.unpack(">Q", blob[:8])
    header = json.loads(blob[8:8 + n])
    body = memoryview(blob)[8 + n:]
    arrays = {}
    for s in header.get("arrays", []):
        arrays[s["name"]] = np.frombuffer(body[s["offset"]:s["offset"] + s["bytes"]],
                                          dtype=np.dtype(s["dtype"])).reshape(s["shape"])
    return header, arrays


def encode_array(a: np.ndarray) -> dict[str, Any]:
    """A small array inside a JSON reply (per-row outputs of a forward call)."""
    import base64
    a = np.ascontiguousarray(a)
    return {"dtype": a.dtype.str, "shape": list(a.shape), "b64": base64.b64encode(a.tobytes()).decode()}


def decode_array(d: dict[str, Any]) -> np.ndarray:
    import base64
    return np.frombuffer(base64.b64decode(d["b64"]), dtype=np.dtype(d["dtype"])).reshape(d["shape"]).copy()


def encode_microbatches(mbs) -> bytes:
    arrays = {}
    for i, mb in enumerate(mbs):
        for name in ("tokens", "targets", "weights", "positions", "cu_seqlens"):
            arrays[f"{i}.{name}"] = getattr(mb, name)
        for name, values in (getattr(mb, "extras", None) or {}).items():
            arrays[f"{i}.extra.{name}"] = values
    extras = sorted((getattr(mbs[0], "extras", None) or {})) if mbs else []
    return encode_arrays({"kind": "microbatches", "count": len(mbs), "extras": extras,
                          "max_seqlen": [int(mb.max_seqlen) for mb in mbs]}, arrays)


def decode_microbatches(blob: bytes):
    from .packing import PackedMicrobatch
    header, arrays = decode_arrays(blob)
    if header.get("kind") != "microbatches":
        raise ValueError("payload is not a microbatch set")
    out = []
    for i in range(header["count"]):
        out.append(PackedMicrobatch(*(np.array(arrays[f"{i}.{n}"]) for n in
                                      ("tokens", "targets", "weights", "positions", "cu_seqlens")),
                                    max_seqlen=header["max_seqlen"][i],
                                    extras={n: np.array(arrays[f"{i}.extra.{n}"])
                                            for n in header.get("extras", [])}))
    return out
