"""Typed save/load on top of the archive container.

``save_artifact(obj, path)`` picks the kind from the object's type;
``load_artifact(path)`` returns the object the archive holds. A ``TensorChunk``
carries a contiguous run of elements of one named tensor as a raw payload, the
unit weights travel in between service and client
(packages/engine/src/shadowspill/artifacts/tensors.py:54-72).
"""
from __future__ import annotations

import os
from dataclasses import asdict, dataclass
from typing import Any

import numpy as np

from .archive import ArtifactError, load_archive, save_archive

_NP = {"bfloat16": np.uint16, "float32": np.float32, "float16": np.float16, "int32": np.int32,
       "int64": np.int64, "uint8": np.uint8}


@dataclass
class TensorChunk:
    name: str
    dtype: str                     # bfloat16 travels as its 16-bit pattern
    shape: tuple[int, ...]         # shape of the whole tensor
    start: int                     # first element of this chunk in the flattened tensor
    data: np.ndarray               # 1-D, dtype _NP[dtype]

    def __post_init__(self) -> None:
        if self.dtype not in _NP:
            raise ArtifactError(f"unsupported tensor dtype {self.dtype!r}")
        self.shape = tuple(int(s) for s in self.shape)
        self.data = np.ascontiguousarray(self.data, dtype=_NP[self.dtype]).reshape(-1)
        total = int(np.prod(self.shape)) if self.shape else 1
        if self.start < 0 or self.start + self.data.size > total:
            raise ArtifactError("chunk lies outside its tensor")


def save_tensor_chunk(chunk: TensorChunk, path: str | os.PathLike) -> None:
    meta = {"name": chunk.name, "dtype": chunk.dtype, "shape": list(chunk.shape),
            "start": chunk.start, "count": int(chunk.data.size)}
    save_archive(path, "tensor_chunk", meta, {"data": chunk.data.tobytes()})


def load_tensor_chunk(path: str | os.PathLike) -> TensorChunk:
    meta, payloads = load_archive(path, "tensor_chunk")
    data = np.frombuffer(payloads["data"], dtype=_NP[meta["dtype"]])
    if data.size != meta["count"]:
        raise ArtifactError("chunk payload has the wrong length")
    return TensorChunk(meta["name"], meta["dtype"], tuple(meta["shape"]), meta["start"], data.copy())


def _kinds() -> dict[str, tuple[type, Any, Any]]:
    from ..communication.info import CommunicationInfo
    from ..communication.measure import PoolMemoryProfile
    from ..ir.plan import Plan
    from ..ir.program import Program
    from ..planning.plan import MemoryBudgets, SweepResult
    from ..profiling.measure import Profiles

    def sweep_to(s: SweepResult) -> dict:
        return {"plans": [None if p is None else p.to_json() for p in s.plans], "errors": s.errors,
                "best": next(i for i, p in enumerate(s.plans) if p is s.best)}

    def sweep_from(d: dict) -> SweepResult:
        plans = [None if p is None else Plan.from_json(p) for p in d["plans"]]
        return SweepResult(plans[d["best"]], plans, list(d["errors"]))

    return {
        "program": (Program, lambda o: o.to_json(), Program.from_json),
        "profiles": (Profiles, lambda o: o.to_json(), Profiles.from_json),
        "plan": (Plan, lambda o: o.to_json(), Plan.from_json),
        "sweep": (SweepResult, sweep_to, sweep_from),
        "budgets": (MemoryBudgets, asdict, lambda d: MemoryBudgets(**d)),
        "communication": (CommunicationInfo, lambda o: o.to_json(), CommunicationInfo.from_json),
        "pool_memory": (PoolMemoryProfile, asdict, lambda d: PoolMemoryProfile(**d)),
    }


def save_artifact(obj: Any, path: str | os.PathLike, max_bytes: int | None = None) -> str:
    """Writes ``obj`` as one archive and returns its kind."""
    if isinstance(obj, TensorChunk):
        save_tensor_chunk(obj, path)
        return "tensor_chunk"
    for kind, (cls, to_json, _) in _kinds().items():
        if isinstance(obj, cls):
            save_archive(path, kind, to_json(obj), max_bytes=max_bytes)
            return kind
    raise TypeError(f"{type(obj).__name__} is not an artifact")


def load_artifact(path: str | os.PathLike, kind: str | None = None) -> Any:
    from .archive import archive_kind
    found = archive_kind(path)
    if kind is not None and found != kind:
        raise ArtifactError(f"archive holds a {found!r}, wanted {kind!r}")
    if found == "tensor_chunk":
        return load_tensor_chunk(path)
    table = _kinds()
    if found not in table:
        raise ArtifactError(f"unknown artifact kind {found!r}")
    meta, _ = load_archive(path, found)
    return table[found][2](meta)
