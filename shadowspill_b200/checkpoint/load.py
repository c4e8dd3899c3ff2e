"""``load_checkpoint`` and layout conversion.

Loading validates the state identity and then copies every owned region into
its spill home. When the saved layout differs from the running one (another
number of data-parallel ranks), each rank assembles its regions from whichever
source archives hold them, so any saved layout restores into any other
(reference: packages/engine/src/shadowspill/checkpoint/{load.py:289,
conversion.py,redistribution.py,mapping.py}).
"""
from __future__ import annotations

from pathlib import Path
from typing import Any

import numpy as np
import torch

from .archive import CheckpointError, iter_members, read_manifest
from .save import state_entries, state_identity

_TORCH = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16,
          "int64": torch.int64, "int32": torch.int32}


def checkpoint_files(directory: str | Path) -> list[Path]:
    files = sorted(Path(directory).glob("rank*.tar"), key=lambda p: int(p.stem[4:]))
    if not files:
        raise CheckpointError(f"{directory}: no rank archives")
    return files


def load_checkpoint(executor, directory: str | Path, strict: bool = True) -> dict[str, Any]:
    """Restores this rank's persistent state; returns the checkpoint metadata."""
    files = checkpoint_files(directory)
    manifests = [read_manifest(f) for f in files]
    saved_world = manifests[0].get("logical_ranks", len(files))
    if len(files) != saved_world:
        raise CheckpointError(f"{directory}: {len(files)} archives for {saved_world} logical ranks")
    mine = state_entries(executor)
    want_identity = state_identity(mine, saved_world)
    if manifests[0]["state"] != want_identity:
        saved = {e["name"]: (e["shape"], e["dtype"]) for e in manifests[0]["tensors"]}
        now = {e["name"]: (e["shape"], e["dtype"]) for e in mine}
        missing = sorted(set(now) - set(saved))[:3]
        extra = sorted(set(saved) - set(now))[:3]
        changed = sorted(k for k in set(now) & set(saved) if now[k] != saved[k])[:3]
        if strict or missing or changed:
            raise CheckpointError(f"{directory}: state identity differs (missing {missing}, "
                                  f"unexpected {extra}, changed {changed})")
    views = dict(executor.named_tensors())
    need = {e["name"]: e for e in mine}
    filled = {name: 0 for name in need}
    for path in files:
        for entry, data in iter_members(path):
            e = need.get(entry["name"])
            if e is None:
                continue
            dt = _TORCH[entry["dtype"]]
            src_lo, src_n = entry["region"]
            dst_lo, dst_n = e["region"]
            lo, hi = max(src_lo, dst_lo), min(src_lo + src_n, dst_lo + dst_n)
            if hi <= lo:
                continue
            src = torch.from_numpy(data.copy()).view(dt)
            dst = views[entry["name"]].reshape(-1)
            dst[lo - dst_lo:hi - dst_lo].copy_(src[lo - src_lo:hi - src_lo])
            filled[entry["name"]] += hi - lo
    short = [n for n, e in need.items() if filled[n] < e["region"][1]]
    if short:
        raise CheckpointError(f"{directory}: regions not covered for {short[:3]}")
    meta = manifests[0].get("metadata", {})
    if "completed_updates" in meta:
        executor.completed_updates = int(meta["completed_updates"])
    return meta


def export_weights(directory: str | Path) -> dict[str, torch.Tensor]:
    """Whole parameters (no optimizer state) assembled from every rank's archive."""
    out: dict[str, torch.Tensor] = {}
    for path in checkpoint_files(directory):
        for entry, data in iter_members(path):
            if entry["name"].startswith(("exp_avg", "master.")):
                continue
            dt = _TORCH[entry["dtype"]]
            full = out.get(entry["name"])
            if full is None:
                full = out[entry["name"]] = torch.zeros(entry["storage_elements"], dtype=dt)
            lo, n = entry["region"]
            full[lo:lo + n].copy_(torch.from_numpy(data.copy()).view(dt)[:n])
    manifest = read_manifest(checkpoint_files(directory)[0])
    shapes = {e["name"]: e["shape"] for e in manifest["tensors"]}
    return {k: v.view(shapes[k]) for k, v in out.items()}
