"""``save_checkpoint``: stream an executor's persistent state into per-rank archives.

Every persistent tensor is read from its home in the pinned spill pool (nothing
is gathered onto a device). A rank writes only the region it owns: the whole
tensor when storage is whole, its slice when storage is sharded. Restore binds
to the *state identity* (names, geometry, owned regions), not to the plan, so a
run with another plan, budget or microbatch geometry can resume from it.

Reference: packages/engine/src/shadowspill/checkpoint/save.py:36,263-291.
"""
from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path
from typing import Any

import numpy as np
import torch

from .archive import FORMAT, VERSION, ArchiveWriter

_NP = {torch.bfloat16: ("bfloat16", np.uint16), torch.float32: ("float32", np.float32),
       torch.float16: ("float16", np.float16), torch.int64: ("int64", np.int64),
       torch.int32: ("int32", np.int32)}


def state_entries(executor) -> list[dict[str, Any]]:
    """Geometry of every persistent tensor as this rank stores it."""
    world, rank = executor.world, executor.rank
    out = []
    for si, st in enumerate(executor.stages):
        for kind, prefix in (("weights", ""), ("exp_avg", "exp_avg."), ("exp_avg_sq", "exp_avg_sq."),
                             ("master", "master.")):
            if f"{st.name}.{kind}" not in executor._obj:
                continue
            for p in st.params:
                if kind != "weights" and not p.trainable:
                    continue          # frozen parameters own no moments and no master copy
                dt = p.dtype or (torch.float32 if kind == "master" else executor.desc.dtype)
                numel, shape = p.numel, p.shape
                if p.expert_sharded:
                    # this rank's experts are rows [expert_lo, expert_lo + local) of the whole bank
                    shape = tuple(p.global_shape)
                    row = p.numel // p.shape[0]
                    numel = row * shape[0]
                    lo, hi = p.expert_lo * row, p.expert_lo * row + p.numel
                else:
                    lo, hi = st.owned_span(p, executor.desc.dtype, world, rank)
                out.append({"name": f"{prefix}{st.name}.{p.name}", "shape": list(shape),
                            "dtype": _NP[dt][0], "stride": _contiguous_stride(shape),
                            "storage_offset": 0, "storage_elements": numel,
                            "region": [lo, hi - lo]})
    return out


def _contiguous_stride(shape) -> list[int]:
    stride, acc = [], 1
    for d in reversed(shape):
        stride.append(acc)
        acc *= d
    return list(reversed(stride))


def state_identity(entries: list[dict[str, Any]], world: int) -> str:
    """Digest of names and geometry, independent of which rank owns what."""
    ident = [[e["name"], e["shape"], e["dtype"]] for e in entries]
    return hashlib.sha256(json.dumps([ident, world], sort_keys=True).encode()).hexdigest()


def save_checkpoint(executor, directory: str | Path, *, metadata: dict[str, Any] | None = None,
                    weights: str = "compute") -> Path:
    """Writes ``<directory>/rank<r>.tar`` for this rank and returns its path."""
    if metadata is not None and len(json.dumps(metadata)) > (16 << 20):
        raise ValueError("checkpoint metadata is limited to 16 MiB of JSON")
    directory = Path(directory)
    if getattr(executor, "replicas", 1) > 1 and executor.global_rank >= executor.world:
        # replicas hold identical state: the first replica's ranks write the checkpoint
        return directory / f"rank{executor.rank}.tar"
    entries = state_entries(executor)
    writer = ArchiveWriter(directory / f"rank{executor.rank}.tar")
    try:
        # streamed: with state homed in a file pool each object is read from the file when its
        # first tensor comes up and dropped again, so one object is in host memory at a time
        by_name = {e["name"]: e for e in entries}
        for name, t in executor.named_tensors(writable=False):
            e = by_name.pop(name, None)
            if e is None:
                continue
            lo, n = e["region"]
            flat = t.reshape(-1)[:n] if executor.world > 1 else t.reshape(-1)
            arr = flat.view(torch.uint8).numpy() if flat.numel() else np.zeros(0, np.uint8)
            writer.add_tensor(e, arr)
            release = getattr(executor, "release_mirrors", None)
            if release is not None:
                release()
        if by_name:
            raise KeyError(f"state tensors without a home: {sorted(by_name)[:3]}")
        manifest = {
            "format": FORMAT, "version": VERSION, "byteorder": sys.byteorder,
            "state": state_identity(entries, executor.world),
            "program": executor.program.digest(), "logical_rank": executor.rank,
            "logical_ranks": executor.world, "additional_programs": [],
            "metadata": dict(metadata or {}, completed_updates=executor.completed_updates),
            "frozen_state_id": None, "omitted_parameters": [], "weights": weights,
            "derived_tensors": [], "gathered_tensors": [], "retained_weight_copies": [],
        }
        return writer.finish(manifest)
    except BaseException:
        writer.abort()
        raise
