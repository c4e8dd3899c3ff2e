"""``load_checkpoint`` and layout conversion.

Loading validates the state identity and then copies every owned region into
its spill home. When the saved layout differs from the running one (another
number of data-parallel ranks), each rank assembles its regions from whichever
source archives hold them, so any saved layout restores into any other
(reference: packages/engine/src/shadowspill/checkpoint/{load.py:289,
conversion.py,redistribution.py,mapping.py}).

A weight held in two precisions is saved once (``weights="master"`` or
``"compute"``); the other copy is listed in the manifest's ``derived_tensors`` and
rebuilt here by a cast (load.py:289 and execution/tensor_copies.py:164 of the
reference). An archive written with a ``frozen_state_id`` holds no frozen parameter
and loads only when the caller names the same id (checkpoint/frozen.py:59-79): the
frozen base then keeps whatever the executor already holds.
"""
from __future__ import annotations

from pathlib import Path
from typing import Any

import torch

from .archive import CheckpointError, iter_members, read_manifest
from .save import (TORCH_DTYPES, derived_tensors, entry_region, omitted_parameters,
                   restore_random_streams, state_entries, state_identity)


def checkpoint_files(directory: str | Path) -> list[Path]:
    files = sorted(Path(directory).glob("rank*.tar"), key=lambda p: int(p.stem[4:]))
    if not files:
        raise CheckpointError(f"{directory}: no rank archives")
    return files


def _saved_world(manifests: list[dict[str, Any]], files: list[Path], directory) -> int:
    first = manifests[0]
    world = first.get("logical_ranks", first.get("metadata", {}).get("logical_ranks", len(files)))
    if len(files) != world:
        raise CheckpointError(f"{directory}: {len(files)} archives for {world} logical ranks")
    ranks = sorted(int(m.get("logical_rank", i)) for i, m in enumerate(manifests))
    if ranks != list(range(world)):
        raise CheckpointError(f"{directory}: logical ranks {ranks} do not cover 0..{world - 1}")
    return int(world)


def load_checkpoint(executor, directory: str | Path, strict: bool = True, *,
                    frozen_state_id: str | None = None, random_streams: bool = True) -> dict[str, Any]:
    """Restores this rank's persistent state; returns the checkpoint metadata."""
    files = checkpoint_files(directory)
    manifests = [read_manifest(f) for f in files]
    first = manifests[0]
    saved_world = _saved_world(manifests, files, directory)
    if first.get("frozen_state_id") != frozen_state_id:
        raise CheckpointError(f"{directory}: checkpoint frozen_state_id differs; supply the same frozen base")
    omit = frozen_state_id is not None
    if omit and first.get("omitted_parameters", []) != omitted_parameters(executor):
        raise CheckpointError(f"{directory}: checkpoint omitted parameter inventory differs")
    weights = first.get("weights", "compute")
    mine = state_entries(executor, omit, weights)
    want_identity = state_identity(mine, saved_world)
    if first["state"] != want_identity:
        geo = lambda e: (list(e["shape"]), str(TORCH_DTYPES[e["dtype"]]))   # noqa: E731
        saved = {e["name"]: geo(e) for e in first["tensors"]}
        now = {e["name"]: geo(e) for e in mine}
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
            dt = TORCH_DTYPES[entry["dtype"]]
            src_lo, src_n = entry_region(entry)
            dst_lo, dst_n = entry_region(e)
            lo, hi = max(src_lo, dst_lo), min(src_lo + src_n, dst_lo + dst_n)
            if hi <= lo:
                continue
            src = torch.from_numpy(data.copy()).view(dt)
            dst = views[entry["name"]].reshape(-1)
            dst[lo - dst_lo:hi - dst_lo].copy_(src[lo - src_lo:hi - src_lo])
            filled[entry["name"]] += hi - lo
    short = [n for n, e in need.items() if filled[n] < entry_region(e)[1]]
    if short:
        raise CheckpointError(f"{directory}: regions not covered for {short[:3]}")
    # the copy that was not saved: master := compute (exact), or compute := round(master)
    for name in derived_tensors(executor, weights):
        if name.startswith("master."):
            views[name].copy_(views[name[len("master."):]].reshape(views[name].shape))
        else:
            views[name].copy_(views["master." + name].reshape(views[name].shape))
    meta = first.get("metadata", {})
    if "completed_updates" in meta:
        executor.completed_updates = int(meta["completed_updates"])
    if random_streams and meta.get("random_streams"):
        mine_meta = next((m.get("metadata", {}) for m in manifests
                          if m.get("logical_rank") == executor.rank), meta)
        restore_random_streams(mine_meta.get("random_streams", []), executor.rank)
    return meta


def export_weights(directory: str | Path) -> dict[str, torch.Tensor]:
    """Whole parameters (no optimizer state) assembled from every rank's archive. With
    ``weights="master"`` archives the fp32 masters are returned under the plain names."""
    out: dict[str, torch.Tensor] = {}
    files = checkpoint_files(directory)
    manifest = read_manifest(files[0])
    masters = manifest.get("weights") == "master"
    derived = set(manifest.get("derived_tensors", []))
    for path in files:
        for entry, data in iter_members(path):
            name = entry["name"]
            if name.startswith("exp_avg"):
                continue
            if name.startswith("master."):
                if not masters or name[len("master."):] not in derived:
                    continue
                name = name[len("master."):]
            dt = TORCH_DTYPES[entry["dtype"]]
            full = out.get(name)
            if full is None:
                full = out[name] = torch.zeros(entry["storage_elements"], dtype=dt)
            lo, n = entry_region(entry)
            full[lo:lo + n].copy_(torch.from_numpy(data.copy()).view(dt)[:n])
    shapes = {e["name"].removeprefix("master."): e["shape"] for e in manifest["tensors"]}
    return {k: v.view(shapes[k]) for k, v in out.items()}
