"""Prepared training bundles: everything the Build / Profile / Communication / Plan phases
produce for one setup, saved as one archive (``training.ssp``) so that a later session,
or every run of a service job, opens the executor directly instead of repeating them.

A bundle is tied to the setup that made it by an identity digest over the model, batch
geometry, budgets, dtype, world size, candidate programs and operations; a session given
a bundle of another identity ignores it and prepares from scratch. The reference keeps
the same four phases as separate processes and bundles their results
(packages/engine/src/shadowspill/training/preparation/phases/operations.py:39-199,
``prepare_job`` in phases/job.py:86).
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import asdict
from pathlib import Path
from typing import Any

from ..artifacts.archive import ArtifactError, load_archive, save_archive
from ..models.config import DecoderConfig

KIND = "training_bundle"
FILE_NAME = "training.ssp"


def setup_identity(setup, cfg: DecoderConfig) -> str:
    """Digest of every setting that changes the programs or their plans (which process runs
    which preparation phase is not one of them)."""
    if hasattr(setup, "__dataclass_fields__") and hasattr(getattr(setup, "optimizer_rule", None), "apply"):
        from dataclasses import replace
        rule = setup.optimizer_rule        # a captured optimizer: its name and constants identify it
        setup = replace(setup, optimizer_rule=f"{rule}:{sorted(rule.defaults.items())}")
    s = asdict(setup) if hasattr(setup, "__dataclass_fields__") else dict(setup)
    keep = {k: s[k] for k in ("device_gib", "spill_gib", "tokens_per_step", "microbatch_tokens", "slots",
                              "mean_seqlen", "dtype", "world_size", "walks", "recompute_shares",
                              "saved_variant", "candidate_selections", "operations", "device",
                              "min_shard_bytes", "head_chunks", "frontend", "axis_chunk_rows", "delta_head_groups", "collective_overhead_us", "master_weights", "optimizer_rule", "spill_pool", "spill_address", "spill_chunk_bytes", "spill_queue_depth")
            if k in s}
    keep["model"] = cfg.to_json()
    keep["search"] = s.get("search")
    blob = json.dumps(keep, sort_keys=True, default=str).encode()
    return hashlib.sha256(blob).hexdigest()


def save_bundle(path: str | Path, identity: str, chosen: int, plan_json: dict, extra_json: dict,
                profiles_json: dict | None, communication_json: dict | None,
                timings: dict[str, float] | None = None) -> Path:
    meta = {"identity": identity, "chosen": int(chosen), "plan": plan_json, "extra_plans": extra_json,
            "profiles": profiles_json, "communication": communication_json,
            "timings": dict(timings or {})}
    return save_archive(path, KIND, meta)


def load_bundle(path: str | Path, identity: str | None = None) -> dict[str, Any] | None:
    """The bundle's contents, or ``None`` when the file is missing, unreadable or was made
    for another setup."""
    p = Path(path)
    if not p.exists():
        return None
    try:
        meta, _ = load_archive(p, KIND)
    except (ArtifactError, OSError, ValueError, KeyError):
        return None
    if identity is not None and meta.get("identity") != identity:
        return None
    return meta
